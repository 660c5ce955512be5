"""Trace-to-file export (reference: ``mim.Export`` / ``ExportFunc``, io/mim/export.go:35-105).

``export(path, module, x)`` runs the module once on ``x`` while the tensor layer reports every
outermost op, translates each op into graph primitives and standard-library calls, stores the
parameters it meets as weights under their module paths (other realized tensors become
constants) and writes weights, metadata and graph into one ``.mim`` file.  Opening the file and
calling ``run`` reproduces the traced computation; an op the graph vocabulary cannot express
fails the export with ``ErrUnsupported`` and names the op.

Shapes are traced as they are; ``dynamic={"x": {0: ("batch", 64)}}`` declares axis 0 of input
``x`` symbolic (any size up to 64) and the symbol is carried through ops whose output keeps that
axis, as the reference's ``ExportOptions`` dynamic axes do.
"""
from __future__ import annotations

import os

from ..tensor import core as C
from ..tensor import errors as E
from . import graph as G

_UNARY_PRIM = {"neg": "neg", "recip": "recip", "sqrt": "sqrt", "sin": "sin"}
_UNARY_CALL = {"exp": "exp.v1", "log": "log.v1", "cos": "cos.v1", "tanh": "tanh.v1", "sigmoid": "sigmoid.v1",
               "erf": "erf.v1", "rsqrt": "rsqrt.v1", "silu": "silu.v1"}


class _Exporter:
    def __init__(self, named_params: dict):
        self.b = G.Builder()
        self.ref: dict = {}           # id(Tensor) -> Ref
        self.keep: list = []          # traced tensors, kept alive so ids stay unique
        self.by_ptr = {}              # (data_ptr, shape, dtype) -> parameter name
        for name, t in named_params.items():
            self.by_ptr[(t.data_ptr(), tuple(t.shape), t.dtype)] = name
        self.n_const = 0
        self.failed = None
        self.sizes: dict = {}         # value index -> sizes seen in the trace

    # ------------------------------------------------------------ operands
    def get(self, t) -> G.Ref:
        """Handle of a traced tensor; an unknown realized tensor becomes a stored weight / constant."""
        r = self.ref.get(id(t))
        if r is not None:
            return r
        if t._val is None:
            raise E.ErrUnsupported(f"export: a value made by {t._opname or 'an op'!r} outside the public tensor ops "
                                   f"cannot be translated")
        from .mim import QuantizedTensor
        val = t._val
        if isinstance(val, QuantizedTensor):
            name = f"qweight.{self.n_const}"
            self.n_const += 1
            r = self.b.weight(name, val)
        else:
            key = (val.data_ptr(), tuple(val.shape), val.dtype)
            name = self.by_ptr.get(key)
            if name is None:
                name, kind = f"const.{self.n_const}", "const"
                self.n_const += 1
            else:
                kind = "weight"
            r = self.b.weight(name, val.detach().cpu().contiguous(), kind)
        self.ref[id(t)] = r
        self.sizes[r.index] = tuple(t.shape)
        self.keep.append(t)
        return r

    def lift(self, x, like: G.Ref) -> G.Ref:
        if isinstance(x, C.Tensor):
            return self.get(x)
        return self.b.const(x, like.dtype, [])

    def put(self, t, r: G.Ref):
        self.ref[id(t)] = r
        self.keep.append(t)

    # --------------------------------------------------------- translation
    def record(self, name, a, k, out):
        if self.failed is not None:
            return
        try:
            self._record(name, a, k, out)
        except E.MimirError as exc:
            self.failed = exc

    def _same_dtype(self, r: G.Ref, t) -> G.Ref:
        want = G.dtype_name(t.dtype)
        return r if r.dtype == want else self.b.cast(r, want)

    def _dims_like(self, out, *srcs):
        """Declared dims of ``out``: its traced sizes, with a symbol wherever a source operand has a
        symbol on the axis that lines up from the right and the traced sizes agree."""
        dims = list(out.shape)
        for s in srcs:
            sd = s.dims
            for i in range(1, min(len(sd), len(dims)) + 1):
                if isinstance(sd[-i], G.Sym) and isinstance(dims[-i], int) and self._traced_size(s, -i) == dims[-i]:
                    dims[-i] = sd[-i]
        return dims

    def _traced_size(self, r: G.Ref, axis):
        return self.sizes[r.index][axis]

    def _record(self, name, a, k, out):
        b = self.b
        outs = out if isinstance(out, (tuple, list)) else (out,)
        if any(isinstance(o, C.Tensor) and o._err is not None for o in outs):
            raise next(o._err for o in outs if isinstance(o, C.Tensor) and o._err is not None)
        r = self._translate(name, a, k, outs)
        if isinstance(r, G.Ref):
            r = [r]
        for o, ref in zip(outs, r):
            self.sizes[ref.index] = tuple(o.shape)
            ref = self._same_dtype(ref, o)
            self.sizes[ref.index] = tuple(o.shape)
            self.put(o, ref)

    def _translate(self, name, a, k, outs):
        b, out = self.b, outs[0]
        T = C.Tensor

        def dims(*srcs):
            return self._dims_like(out, *srcs)

        def dt():
            return G.dtype_name(out.dtype)

        def f(x, like=None):
            return self.get(x) if isinstance(x, T) else b.const(x, (like.dtype if like is not None else dt()), [])

        if name in _UNARY_PRIM:
            x = self.get(a[0])
            return b.op(_UNARY_PRIM[name], [x], [(x.dtype, dims(x))])[0]
        if name in _UNARY_CALL:
            x = self.get(a[0])
            return b.call1(_UNARY_CALL[name], [x], dt(), dims(x))
        if name == "relu":
            x = self.get(a[0])
            return b.op("max", [x, b.const(0, x.dtype, [])], [(x.dtype, dims(x))])[0]
        if name == "gelu":
            x = self.get(a[0])
            approx = k.get("approximate", a[1] if len(a) > 1 else "tanh")
            return b.call1("gelu_tanh.v1" if approx == "tanh" else "gelu_erf.v1", [x], dt(), dims(x))
        if name in ("abs_", "abs"):
            x = self.get(a[0])
            neg = b.op("neg", [x], [(x.dtype, dims(x))])[0]
            return b.op("max", [x, neg], [(x.dtype, dims(x))])[0]
        if name == "leaky_relu":
            x = self.get(a[0])
            slope = k.get("slope", a[1] if len(a) > 1 else 0.01)
            neg = b.op("mul", [x, b.const(float(slope), x.dtype, [])], [(x.dtype, dims(x))])[0]
            return b.op("max", [x, neg], [(x.dtype, dims(x))])[0] if slope <= 1 else \
                b.op("where", [b.op("cmplt", [x, b.const(0, x.dtype, [])], [("i32", dims(x))])[0], neg, x],
                     [(x.dtype, dims(x))])[0]
        if name in ("add", "mul", "maximum", "pow_", "sub", "div", "minimum"):
            like = self.get(a[0]) if isinstance(a[0], T) else self.get(a[1])
            x, y = f(a[0], like), f(a[1], like)
            want = dt()
            if x.dtype != want:
                x = self._cast(x, want)
            if y.dtype != want:
                y = self._cast(y, want)
            d = dims(x, y)
            if name == "sub":
                y = b.op("neg", [y], [(want, y.dims)])[0]
                return b.op("add", [x, y], [(want, d)])[0]
            if name == "div":
                if want not in ("f32", "f16", "bf16", "f64"):
                    return b.op("idiv", [x, y], [(want, d)])[0]
                y = b.op("recip", [y], [(want, y.dims)])[0]
                return b.op("mul", [x, y], [(want, d)])[0]
            if name == "minimum":
                nx = b.op("neg", [x], [(want, x.dims)])[0]
                ny = b.op("neg", [y], [(want, y.dims)])[0]
                m = b.op("max", [nx, ny], [(want, d)])[0]
                return b.op("neg", [m], [(want, d)])[0]
            code = {"add": "add", "mul": "mul", "maximum": "max", "pow_": "pow"}[name]
            return b.op(code, [x, y], [(want, d)])[0]
        if name in ("less", "equal"):
            like = self.get(a[0]) if isinstance(a[0], T) else self.get(a[1])
            x, y = f(a[0], like), f(a[1], like)
            if x.dtype != y.dtype:
                y = self._cast(y, x.dtype)
            r = b.op("cmplt" if name == "less" else "cmpeq", [x, y], [("i32", dims(x, y))])[0]
            return r
        if name in ("logical_and", "logical_or"):
            # truth values are the i32 0 / 1 that comparisons give; any other operand is first compared with zero
            def truth(v):
                t = self.get(v)
                if t.dtype == "i32":
                    return t
                isz = b.op("cmpeq", [t, b.const(0, t.dtype, [])], [("i32", dims(t))])[0]
                self.sizes[isz.index] = self.sizes[t.index]
                r = b.op("cmpeq", [isz, b.const(0, "i32", [])], [("i32", dims(t))])[0]
                self.sizes[r.index] = self.sizes[t.index]
                return r
            x, y = truth(a[0]), truth(a[1])
            return b.op("and" if name == "logical_and" else "or", [x, y], [("i32", dims(x, y))])[0]
        if name == "logical_not":
            x = self.get(a[0])
            return b.op("cmpeq", [x, b.const(0, x.dtype, [])], [("i32", dims(x))])[0]
        if name == "where":
            c = self.get(a[0])
            like = self.get(a[1]) if isinstance(a[1], T) else (self.get(a[2]) if isinstance(a[2], T) else None)
            x, y = f(a[1], like), f(a[2], like)
            want = dt()
            x, y = (self._cast(x, want) if x.dtype != want else x), (self._cast(y, want) if y.dtype != want else y)
            return b.op("where", [c, x, y], [(want, dims(c, x, y))])[0]
        if name == "cast":
            x = self.get(a[0])
            return self._cast(x, G.dtype_name(out.dtype))
        if name in ("reshape", "squeeze", "unsqueeze", "contiguous"):
            x = self.get(a[0])
            if name == "contiguous":
                return x
            return b.op("reshape", [x], [(x.dtype, self._reshape_dims(x, out))])[0]
        if name == "permute":
            x = self.get(a[0])
            perm = [p % len(x.dims) for p in (k.get("dims") if "dims" in k else a[1])]
            return b.op("permute", [x], [(x.dtype, [x.dims[p] for p in perm])], perm=perm)[0]
        if name == "transpose":
            x = self.get(a[0])
            n = len(x.dims)
            p, q = (list(a[1:]) + [-1, -2][len(a) - 1:])[:2] if len(a) > 1 else (k.get("a", -1), k.get("b", -2))
            perm = list(range(n))
            perm[p % n], perm[q % n] = perm[q % n], perm[p % n]
            return b.op("permute", [x], [(x.dtype, [x.dims[i] for i in perm])], perm=perm)[0]
        if name == "expand":
            x = self.get(a[0])
            return b.op("expand", [x], [(x.dtype, dims(x))])[0]
        if name == "pad":
            x = self.get(a[0])
            return b.pad(x, [tuple(p) for p in a[1]], k.get("value", a[2] if len(a) > 2 else 0.0))
        if name == "shrink":
            x = self.get(a[0])
            return b.shrink(x, [tuple(p) for p in a[1]])
        if name == "getitem":
            return self._getitem(self.get(a[0]), a[1], out)
        if name == "cat":
            return self._cat([self.get(t) for t in a[0]], k.get("dim", a[1] if len(a) > 1 else 0), out)
        if name in ("sum_", "max_", "mean", "min_"):
            return self._reduce(name, self.get(a[0]), k.get("dim", a[1] if len(a) > 1 else None),
                                k.get("keepdim", a[2] if len(a) > 2 else False), out)
        if name in ("softmax", "log_softmax"):
            x = self.get(a[0])
            axis = k.get("dim", a[1] if len(a) > 1 else -1)
            return b.call1(name + ".v1", [x], dt(), dims(x), axis=int(axis))
        if name == "matmul":
            x, y = self.get(a[0]), self.get(a[1])
            d = list(out.shape)
            for i in range(len(d) - 1):
                src = x.dims if len(x.dims) >= len(y.dims) else y.dims
                j = i - (len(d) - len(src))
                if 0 <= j < len(src) - 1 and isinstance(src[j], G.Sym):
                    d[i] = src[j]
            return b.call1("matmul.v1", [x, y], dt(), d)
        if name == "matmul_t":
            x = self.get(a[0])
            w = a[1]
            from .mim import QuantizedTensor
            bias = k.get("bias", a[2] if len(a) > 2 else None)
            ins = [x]
            d = x.dims[:-1] + [out.shape[-1]]
            if isinstance(w, QuantizedTensor):
                nm = f"qweight.{self.n_const}"
                self.n_const += 1
                ins.append(b.weight(nm, w))
                if bias is not None:
                    ins.append(self.get(bias))
                return b.call1("dequant_matmul.v1", ins, dt(), d)
            ins.append(self.get(w))
            if bias is not None:
                ins.append(self.get(bias))
            return b.call1("linear.v1", ins, dt(), d)
        if name == "layer_norm":
            x = self.get(a[0])
            w = k.get("weight", a[1] if len(a) > 1 else None)
            bias = k.get("bias", a[2] if len(a) > 2 else None)
            eps = k.get("eps", a[3] if len(a) > 3 else 1e-5)
            ins = [x]
            if w is None and bias is not None:
                ins.append(b.const(1.0, x.dtype, []))
            if w is not None:
                ins.append(self.get(w))
            if bias is not None:
                ins.append(self.get(bias))
            return b.call1("layer_norm.v1", ins, dt(), dims(x), axes=[-1], eps=float(eps))
        if name == "rms_norm":
            x = self.get(a[0])
            w = k.get("weight", a[1] if len(a) > 1 else None)
            eps = k.get("eps", a[2] if len(a) > 2 else 1e-6)
            ins = [x] + ([self.get(w)] if w is not None else [])
            return b.call1("rms_norm.v1", ins, dt(), dims(x), axes=[-1], eps=float(eps), round_before_scale=True)
        if name == "swiglu":
            g_, u = self.get(a[0]), self.get(a[1])
            return b.call1("swiglu.v1", [g_, u], dt(), dims(g_, u))
        if name == "gather_rows":
            table, idx = self.get(a[0]), self.get(a[1])
            return b.call1("embedding.v1", [table, idx], dt(), idx.dims + table.dims[1:])
        if name == "conv2d":
            x, w = self.get(a[0]), self.get(a[1])
            names = ("bias", "stride", "padding", "dilation", "groups")
            defaults = (None, 1, 0, 1, 1)
            vals = {n: k.get(n, a[2 + i] if len(a) > 2 + i else defaults[i]) for i, n in enumerate(names)}
            pair = lambda v: [int(v), int(v)] if isinstance(v, int) else [int(i) for i in v]
            ins = [x, w] + ([self.get(vals["bias"])] if vals["bias"] is not None else [])
            p = pair(vals["padding"])
            d = [x.dims[0]] + list(out.shape[1:])
            return b.call1("conv2d.v1", ins, dt(), d, strides=pair(vals["stride"]), dilations=pair(vals["dilation"]),
                           pads=[p[0], p[0], p[1], p[1]], groups=int(vals["groups"]))
        if name == "attention":
            q, kk, v = self.get(a[0]), self.get(a[1]), self.get(a[2])
            names = ("causal", "causal_offset", "mask", "scale")
            defaults = (False, None, None, None)
            vals = {n: k.get(n, a[3 + i] if len(a) > 3 + i else defaults[i]) for i, n in enumerate(names)}
            tq, tk = a[0].shape[2], a[1].shape[2]
            if vals["causal"] and vals["causal_offset"] not in (None, tk - tq):
                raise E.ErrUnsupported("export: attention with a causal offset other than keys - queries")
            ins = [q, kk, v] + ([self.get(vals["mask"])] if vals["mask"] is not None else [])
            return b.call1("attention.v1", ins, dt(), dims(q), causal=bool(vals["causal"]),
                           scale=float(vals["scale"] or 0.0))
        if name == "cumsum":
            x = self.get(a[0])
            return b.call1("cumsum.v1", [x], dt(), dims(x), axis=int(k.get("dim", a[1] if len(a) > 1 else -1)))
        if name == "argsort":
            x = self.get(a[0])
            r = b.call1("argsort.v1", [x], "i64", dims(x), axis=int(k.get("dim", a[1] if len(a) > 1 else -1)),
                        descending=bool(k.get("descending", a[2] if len(a) > 2 else False)))
            return r
        if name == "topk":
            x = self.get(a[0])
            kk = int(k.get("k", a[1] if len(a) > 1 else 1))
            axis = int(k.get("dim", a[2] if len(a) > 2 else -1))
            d = x.dims[:]
            d[axis % len(d)] = kk
            largest = bool(k.get("largest", a[3] if len(a) > 3 else True))
            return b.call("top_k.v1", [x], [(x.dtype, d), ("i64", d)], k=kk, axis=axis, largest=largest)
        if name in ("zeros", "ones", "full"):
            value = 0 if name == "zeros" else 1 if name == "ones" else k.get("value", a[1] if len(a) > 1 else 0)
            return b.const(value, dt(), list(out.shape))
        from .export_decompose import REWRITES
        rewrite = REWRITES.get(name)
        if rewrite is not None:
            # rebuilt from ops that have translations; the trace is live, so the rebuild is recorded as it runs
            res = rewrite(*a, **k)
            if isinstance(res, (tuple, list)):
                return [self.get(r) for r in res]
            return self.get(res)
        raise E.ErrUnsupported(f"export: op {name!r} has no translation into the graph vocabulary")

    def _cast(self, x, dtype):
        r = self.b.cast(x, dtype)
        self.sizes[r.index] = self.sizes.get(x.index, ())
        return r

    def _reshape_dims(self, x, out):
        """Carries symbolic axes through a reshape that keeps them whole: an axis of the operand whose traced
        size reappears at the same offset (the product of the sizes before it) in the result stays symbolic
        there, wherever it lands (``[batch, F] -> [1, batch, F]`` as well as ``[batch, a, b] -> [batch, a * b]``)."""
        d = list(out.shape)
        sx = tuple(self.sizes.get(x.index, ()))
        if len(sx) != len(x.dims):
            return d
        before = 1
        for i, dim in enumerate(x.dims):
            if isinstance(dim, G.Sym):
                acc = 1
                for j, size in enumerate(d):
                    if acc == before and size == sx[i] and not isinstance(d[j], G.Sym):
                        d[j] = dim
                        break
                    acc *= size if isinstance(size, int) else 1
                    if acc > before:
                        break
            before *= sx[i]
        return d

    def _getitem(self, x, idx, out):
        b = self.b
        if not isinstance(idx, tuple):
            idx = (idx,)
        if any(i is Ellipsis for i in idx):
            n = len(x.dims) - (len(idx) - 1 - sum(i is None for i in idx))
            j = idx.index(Ellipsis)
            idx = idx[:j] + (slice(None),) * n + idx[j + 1:]
        sizes = self.sizes[x.index]
        ranges, ax = [], 0
        for i in idx:
            if i is None:
                continue
            n = sizes[ax]
            if isinstance(i, int):
                i = i % n
                ranges.append((i, i + 1))
            elif isinstance(i, slice):
                lo, hi, st = i.indices(n)
                if st != 1:
                    raise E.ErrUnsupported("export: a slice with a step")
                if (lo, hi) == (0, n):
                    ranges.append((0, -1))
                else:
                    ranges.append((lo, max(hi, lo)))
            else:
                raise E.ErrUnsupported(f"export: index of type {type(i).__name__}")
            ax += 1
        ranges += [(0, -1)] * (len(x.dims) - len(ranges))
        r = b.shrink(x, ranges) if any(rg != (0, -1) for rg in ranges) else x
        self.sizes[r.index] = tuple((n if hi == -1 else hi) - lo for n, (lo, hi) in zip(sizes, ranges))
        if tuple(self.sizes[r.index]) != tuple(out.shape):
            d = self._reshape_dims(r, out)
            r = b.op("reshape", [r], [(r.dtype, d)])[0]
        return r

    def _cat(self, xs, dim, out):
        """Concatenation as pads plus adds: each part is padded with zeros to the full length along
        the axis and the padded parts are summed (the reference's exporter does the same)."""
        b = self.b
        n = len(out.shape)
        dim %= n
        total = out.shape[dim]
        at, acc = 0, None
        for x in xs:
            size = self.sizes[x.index][dim]
            pads = [(0, 0)] * n
            pads[dim] = (at, total - at - size)
            if x.dtype == "bool":
                raise E.ErrUnsupported("export: cat of bool tensors")
            p = b.pad(x, pads, 0.0)
            self.sizes[p.index] = tuple(out.shape)
            acc = p if acc is None else b.op("add", [acc, p], [(p.dtype, p.dims)])[0]
            at += size
        return acc

    def _reduce(self, name, x, dim, keepdim, out):
        b = self.b
        n = len(x.dims)
        axes = list(range(n)) if dim is None else [d % n for d in ([dim] if isinstance(dim, int) else list(dim))]
        kept = [1 if i in axes else d for i, d in enumerate(x.dims)]
        src = x
        if x.dtype in ("f16", "bf16"):
            src = self._cast(x, "f32")
        if name == "mean":
            r = b.call1("mean.v1", [src], src.dtype, kept, axes=axes, keepdims=True)
        elif name == "min_":
            ng = b.op("neg", [src], [(src.dtype, src.dims)])[0]
            r = b.op("reduce", [ng], [(src.dtype, kept)], mode="max", axes=axes)[0]
            r = b.op("neg", [r], [(src.dtype, kept)])[0]
        else:
            r = b.op("reduce", [src], [(src.dtype, kept)], mode="add" if name == "sum_" else "max", axes=axes)[0]
        if not (keepdim and dim is not None):
            final = [d for i, d in enumerate(kept) if i not in axes] if dim is not None else []
            r = b.op("reshape", [r], [(r.dtype, final)])[0]
        return r


def _named_params(module) -> dict:
    out = {}
    if module is not None and hasattr(module, "named_params"):
        for name, p in module.named_params():
            out[name] = p.value().data()
    return out


def export_func(path, fn, args, input_names=None, output_names=None, dynamic=None, metadata=None, module=None):
    """Traces ``fn(*args)`` (tensors in, a tensor or a sequence of tensors out) and writes the file.
    ``path`` may be a file name or a writable binary stream.  Returns the ``Graph``."""
    args = [a if isinstance(a, C.Tensor) else C.from_torch(a) for a in args]
    names = list(input_names or [f"input{i}" if len(args) > 1 else "input" for i in range(len(args))])
    ex = _Exporter(_named_params(module))
    dynamic = dynamic or {}
    for name, a in zip(names, args):
        if a.err is not None:
            raise a.err
        dims = list(a.shape)
        for axis, (sym, bound) in (dynamic.get(name) or {}).items():
            if a.shape[axis] > bound:
                raise E.ErrShape(f"export: input {name!r} has {a.shape[axis]} along dynamic axis {axis}, bound {bound}")
            dims[axis] = G.Sym(sym, int(bound))
        r = ex.b.input(name, a.dtype, dims)
        ex.sizes[r.index] = tuple(a.shape)
        ex.put(a, r)
    was_training = getattr(module, "training", None)
    if module is not None and hasattr(module, "eval"):
        module.eval()
    try:
        with C.trace_ops(ex.record):
            outs = fn(*args)
    finally:
        if module is not None and was_training and hasattr(module, "train"):
            module.train()
    if ex.failed is not None:
        raise ex.failed
    if isinstance(outs, C.Tensor):
        outs = [outs]
    onames = list(output_names or [f"output{i}" if len(outs) > 1 else "output" for i in range(len(outs))])
    for name, o in zip(onames, outs):
        if o.err is not None:
            raise o.err
        ex.b.output(name, ex.get(o))
    md = dict(metadata or {})
    md.setdefault("format.producer", "mimir_b200")
    if hasattr(path, "write"):
        path.write(ex.b.serialize(metadata=md))
    else:
        ex.b.write(os.fspath(path), metadata=md)
    return ex.b.g


def export(path, module, x, input_name="input", output_name="output", dynamic=None, metadata=None):
    """Exports ``module`` traced on the example input ``x`` (reference: mim.Export).  The module is
    put in evaluation mode for the trace, so dropout is the identity and batch norm uses its running
    statistics."""
    return export_func(path, lambda t: module(t), [x], [input_name], [output_name], dynamic, metadata, module)
