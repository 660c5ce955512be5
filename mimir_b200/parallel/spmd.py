"""The partitioner: any lazy graph over a device mesh, SPMD style.

The reference shards ONE lazy graph over the devices of a mesh in two passes
(tensor/partition.go:131-190 analyse, :341-492 lower): per-op *layout rules*
(tensor/layout.go:229-386, matmul :629-714, attention :832-888) give every value a layout
(each tensor dimension split over a mesh axis or not, plus the axes over which the local
value is only a partial sum), and *conversions* between layouts become collectives
(tensor/reshard.go:86-336: all-reduce or reduce-scatter of partial sums, one all-gather, a
local cut).  This module is that machinery for one process per device:

* ``Layout`` is the state of a value on the mesh; ``rule_for`` is the rules table.
* ``analyse`` walks a graph of *global-shape* lazy tensors whose leaves carry layouts
  (sharded inputs made by ``place``, parameters sharded by ``shard_params``) and decides,
  per node, the layouts it needs from its operands and the layout it produces.  Analyses
  are cached by graph structure (tensor/plancache.go:35-215).
* ``lower`` rebuilds the graph node by node on this rank's blocks, with the same public
  op constructors a single-device graph uses, inserting conversions where an operand's
  layout differs from the one needed.  A conversion of one (node, layout) pair is made
  once and shared (a weight gathered by the forward pass is reused by backward).
* Conversions are differentiable: all-gather <-> cut, all-reduce of partials <-> identity,
  reduce-scatter <-> all-gather.  A replicated value that meets operands split over a mesh
  axis gets an identity whose gradient is all-reduced over that axis (so every cotangent has
  the layout of its value); where that follows an all-gather the pair is one collective:
  all-gather forward, reduce-scatter backward: the fully sharded weight pattern
  (tensor/reshard.go:175-184).

With it a model needs no sharded layer classes: ``nn.Embedding``, ``LayerNorm``, a reshape that
carries a split, attention over sharded heads and a loss over a ``P("data")`` batch all follow
from the rules.  Collectives are ``torch.distributed`` calls on the mesh's axis groups and are
counted in ``Mesh.traffic`` like ``Mesh.Traffic`` (tensor/mesh.go:66-96).  There is no
all-to-all: a split that moves from one axis to another is gathered and cut again, as in the
reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import tensor as T
from ..tensor import core as C
from .mesh import Mesh, PartitionSpec


# =========================================================================== layouts
@dataclass(frozen=True)
class Layout:
    """``dims[d]`` = mesh axis that splits tensor dimension d (or None); ``sections[d]`` = sizes of
    the sections a fused dimension is split by, each section cut on its own ([Q | K | V] rows);
    ``partial`` = axes over which the local block is a partial sum of the value."""
    dims: tuple
    partial: frozenset = frozenset()
    sections: tuple = ()          # ((dim, sizes), ...)

    def axes(self) -> set:
        return {a for a in self.dims if a is not None} | set(self.partial)

    def section_of(self, d: int):
        for dd, sizes in self.sections:
            if dd == d:
                return sizes
        return None

    def resolved(self) -> "Layout":
        return Layout(self.dims, frozenset(), self.sections)

    def replicated(self) -> "Layout":
        return Layout((None,) * len(self.dims))

    @staticmethod
    def of_spec(spec: PartitionSpec | None, ndim: int) -> "Layout":
        if spec is None:
            return Layout((None,) * ndim)
        dims = tuple(spec) + (None,) * (ndim - len(spec))
        sec = ((spec.sections[0], tuple(spec.sections[1])),) if getattr(spec, "sections", None) else ()
        return Layout(dims[:ndim], frozenset(), sec)


def local_shape(shape, lay: Layout, mesh: Mesh) -> tuple:
    return tuple(s // mesh.axis_size(a) if a is not None else s for s, a in zip(shape, lay.dims))


# =========================================================================== differentiable collectives
def _regroup_sections(full, d, sizes, n):
    """An all-gathered sectioned dimension comes out [rank][section]; the value's order is [section][rank]."""
    per = [s // n for s in sizes]
    blocks = full.split([p for _ in range(n) for p in per], d)
    return torch.cat([blocks[r * len(per) + s] for s in range(len(per)) for r in range(n)], d)


def _cut(v, mesh, axis, d, sizes):
    n, i = mesh.axis_size(axis), mesh.axis_index(axis)
    if sizes is None:
        per = v.shape[d] // n
        return v.narrow(d, i * per, per)
    parts, off = [], 0
    for s in sizes:
        parts.append(v.narrow(d, off + i * (s // n), s // n))
        off += s
    return torch.cat(parts, d)


def _gather(v, mesh, axis, d, sizes):
    full = mesh.all_gather(v, axis, d)
    return full if sizes is None else _regroup_sections(full, d, sizes, mesh.axis_size(axis))


def _scatter_sum(v, mesh, axis, d, sizes):
    """Sum over the ranks of ``axis``, each keeping its block of dimension d."""
    n = mesh.axis_size(axis)
    if sizes is not None:      # bring the blocks of one rank together before the plain reduce-scatter
        per = [s // n for s in sizes]
        blocks = v.split([p for s in per for p in [s] * n], d)      # [section][rank]
        v = torch.cat([blocks[s * n + r] for r in range(n) for s in range(len(per))], d)
    return mesh.reduce_scatter(v.contiguous(), axis, d)


class _AllReduce(torch.autograd.Function):          # partial -> whole; cotangent passes through
    @staticmethod
    def forward(ctx, v, mesh, axis, op):
        return mesh.all_reduce(v, axis, op)

    @staticmethod
    def backward(ctx, g):
        return g, None, None, None


class _Mark(torch.autograd.Function):               # identity; the cotangent is summed over the axis
    @staticmethod
    def forward(ctx, v, mesh, axis):
        ctx.m = (mesh, axis)
        return v.view_as(v)

    @staticmethod
    def backward(ctx, g):
        mesh, axis = ctx.m
        return mesh.all_reduce(g.contiguous(), axis), None, None


class _AllGather(torch.autograd.Function):          # split -> whole; cotangent: cut, or (marked) reduce-scatter
    @staticmethod
    def forward(ctx, v, mesh, axis, d, sizes, marked):
        ctx.m = (mesh, axis, d, sizes, marked)
        return _gather(v, mesh, axis, d, sizes)

    @staticmethod
    def backward(ctx, g):
        mesh, axis, d, sizes, marked = ctx.m
        out = _scatter_sum(g, mesh, axis, d, sizes) if marked else _cut(g, mesh, axis, d, sizes).contiguous()
        return out, None, None, None, None, None


class _Cut(torch.autograd.Function):                # whole -> split (no traffic); cotangent: all-gather
    @staticmethod
    def forward(ctx, v, mesh, axis, d, sizes):
        ctx.m = (mesh, axis, d, sizes)
        return _cut(v, mesh, axis, d, sizes).contiguous()

    @staticmethod
    def backward(ctx, g):
        mesh, axis, d, sizes = ctx.m
        return _gather(g.contiguous(), mesh, axis, d, sizes), None, None, None, None


class _ReduceScatter(torch.autograd.Function):      # partial -> split; cotangent: all-gather
    @staticmethod
    def forward(ctx, v, mesh, axis, d, sizes):
        ctx.m = (mesh, axis, d, sizes)
        return _scatter_sum(v, mesh, axis, d, sizes)

    @staticmethod
    def backward(ctx, g):
        mesh, axis, d, sizes = ctx.m
        return _gather(g.contiguous(), mesh, axis, d, sizes), None, None, None, None


def _lazy(fn_real, meta_shape, x: C.Tensor, name: str) -> C.Tensor:
    def run(v):
        if v.device.type == "meta":
            return torch.empty(meta_shape(tuple(v.shape)), dtype=v.dtype, device="meta")
        return fn_real(v)
    return C._node(run, (x,), {}, name)


def _scaled(shape, d, f):
    s = list(shape)
    s[d] = int(s[d] * f) if f >= 1 else s[d] // int(round(1 / f))
    return tuple(s)


def convert(x: C.Tensor, src: Layout, dst: Layout, mesh: Mesh, marks=frozenset()) -> C.Tensor:
    """``x`` (a local lazy tensor in layout ``src``) in layout ``dst``; at most one collective per
    partial axis and per re-split dimension.  ``marks``: axes over which the consumer's output is
    split while ``dst`` is not, so the cotangent has to be summed over them."""
    marks = set(marks)
    # 1. partial sums: reduce-scatter onto a dimension the target splits over that axis, else all-reduce
    for a in sorted(src.partial - dst.partial):
        n = mesh.axis_size(a)
        tgt = [d for d, ax in enumerate(dst.dims) if ax == a and src.dims[d] is None]
        if tgt and n > 1:
            d, sizes = tgt[0], dst.section_of(tgt[0])
            x = _lazy(lambda v, a=a, d=d, sizes=sizes: _ReduceScatter.apply(v, mesh, a, d, sizes),
                      lambda s, d=d, n=n: _scaled(s, d, 1.0 / n), x, "reduce_scatter")
            src = Layout(tuple(a if i == d else ax for i, ax in enumerate(src.dims)), src.partial - {a},
                         src.sections + (((d, sizes),) if sizes else ()))
        else:
            if n > 1:
                x = _lazy(lambda v, a=a: _AllReduce.apply(v, mesh, a, "sum"), lambda s: s, x, "all_reduce")
            src = Layout(src.dims, src.partial - {a}, src.sections)
    # 2. dimensions split differently: gather what the target does not split that way, then cut
    for d, (sa, da) in enumerate(zip(src.dims, dst.dims)):
        if sa == da and src.section_of(d) == dst.section_of(d):
            continue
        if sa is not None:
            n, sizes = mesh.axis_size(sa), src.section_of(d)
            marked = sa in marks and sa not in dst.axes()
            if n > 1:
                x = _lazy(lambda v, sa=sa, d=d, sizes=sizes, marked=marked: _AllGather.apply(v, mesh, sa, d, sizes, marked),
                          lambda s, d=d, n=n: _scaled(s, d, n), x, "all_gather")
            if marked:
                marks.discard(sa)
        if da is not None:
            n, sizes = mesh.axis_size(da), dst.section_of(d)
            if n > 1:
                x = _lazy(lambda v, da=da, d=d, sizes=sizes: _Cut.apply(v, mesh, da, d, sizes),
                          lambda s, d=d, n=n: _scaled(s, d, 1.0 / n), x, "cut")
    # 3. cotangents that come back partial over an axis this value is whole on
    for a in sorted(marks):
        if a not in dst.axes() and mesh.axis_size(a) > 1 and x.dtype.is_floating_point:
            x = _lazy(lambda v, a=a: _Mark.apply(v, mesh, a), lambda s: s, x, "mark")
    return x


# =========================================================================== leaves on the mesh
class MeshTensor(C.Tensor):
    """A leaf of a sharded graph: global shape, this rank's block, its layout."""

    def __init__(self, local: torch.Tensor, shape, mesh: Mesh, layout: Layout, param=None):
        super().__init__(val=None, shape=tuple(shape), dtype=local.dtype, device=C._dev_of(local))
        self.local, self.mesh, self.layout, self.param = local, mesh, layout, param
        self._sharding = (mesh, layout)


def place(x, mesh: Mesh, spec: PartitionSpec | None = None, local: bool = False) -> MeshTensor:
    """A tensor on the mesh.  ``x`` is the whole value (every rank passes the same one and keeps its
    block) or, with ``local=True``, already this rank's block of it."""
    v = x.data() if isinstance(x, C.Tensor) else torch.as_tensor(x)
    if local:
        lay = Layout.of_spec(spec, v.dim())
        shape = tuple(s * mesh.axis_size(a) if a is not None else s for s, a in zip(v.shape, lay.dims))
        return MeshTensor(v, shape, mesh, lay)
    lay = Layout.of_spec(spec, v.dim())
    blk = v
    for d, a in enumerate(lay.dims):
        if a is not None:
            if v.shape[d] % mesh.axis_size(a):
                raise T.ErrShape(f"dimension {d} of size {v.shape[d]} does not split {mesh.axis_size(a)} ways")
            blk = _cut(blk, mesh, a, d, lay.section_of(d))
    return MeshTensor(blk.contiguous(), v.shape, mesh, lay)


def shard_params(model, mesh: Mesh, rule=None, data_axis: str = "data"):
    """Gives every parameter of ``model`` a layout on ``mesh`` (``rule`` as in ``parallel.mesh``:
    ``tensor_parallel``, ``fully_shard``, ``rules``; None = replicated) and keeps only its local
    block.  ``Param.value()`` then returns a mesh leaf, and any graph built from it is partitioned."""
    from ..nn.module import Linear
    from .mesh import _owner_module
    for name, p in model.named_params():
        spec = rule.match(name, p, mesh) if rule is not None else None
        owner = _owner_module(model, name)
        if spec is not None and isinstance(owner, Linear) and getattr(owner, "_qkv_sections", None) \
                and spec[0] is not None and spec[0] != data_axis:
            spec = spec.with_sections(0, *owner._qkv_sections)
        full = p._data
        lay = Layout.of_spec(spec, full.dim())
        blk = full
        for d, a in enumerate(lay.dims):
            if a is not None:
                blk = _cut(blk, mesh, a, d, lay.section_of(d))
        p._full_shape = tuple(full.shape)
        p._data = blk.contiguous().clone()
        p._spmd = (mesh, lay)
        p._mesh, p._spec = mesh, spec          # what parallel.mesh.gather_param reads
        p._version += 1
    model._mesh = mesh
    return model


def _param_leaf(p) -> MeshTensor:
    mesh, lay = p._spmd
    t = MeshTensor(p._data, p._full_shape, mesh, lay, param=p)
    return t


# =========================================================================== rules
_LINEAR_UNARY = {"neg", "cast", "detach", "contiguous", "with_effects", "to"}
_NONLINEAR_UNARY = {"exp", "log", "sqrt", "rsqrt", "sin", "cos", "tanh", "sigmoid", "relu", "abs", "sign", "floor", "ceil",
                    "recip", "erf", "erfinv", "log1p", "expm1", "lgamma", "digamma", "logical_not", "silu", "softplus",
                    "gelu", "leaky_relu", "clamp", "trigamma"}
_BINARY = {"add", "sub", "mul", "div", "maximum", "minimum", "pow", "less", "equal", "mod", "swiglu", "where"}
_MEAN_LOSSES = {"mse", "l1", "huber", "smooth_l1", "bce", "bce_with_logits"}
_ROW_LOSSES = {"cross_entropy", "nll", "label_smoothing", "focal"}


class _Plan:
    """What ``analyse`` decides for one node: the layout each tensor operand must arrive in, the
    layout of the result, and optionally a function that builds the local node(s)."""
    __slots__ = ("needs", "out", "build")

    def __init__(self, needs, out, build=None):
        self.needs, self.out, self.build = needs, out, build


def _merge_axis(cands, used):
    for a in cands:
        if a is not None and a not in used:
            return a
    return None


def _rule_elementwise(node, ins, lays, mesh):
    """Broadcasting elementwise ops.  A sum over ranks passes through the ops that are linear in the
    partial operand (add / sub of equally partial values, mul / div by a whole value); everything
    else first makes its operands whole."""
    nd = len(node.shape)
    op = node._opname
    tens = [i for i, a in enumerate(ins) if isinstance(a, C.Tensor)]
    parts = [lays[i].partial for i in tens]
    keep = frozenset()
    if len(tens) == 2:
        if op in ("add", "sub") and parts[0] == parts[1]:
            keep = parts[0]                                  # sum of sums
        elif op == "mul" and bool(parts[0]) != bool(parts[1]):
            keep = parts[0] or parts[1]                      # (sum of a_r) * c = sum of (a_r * c)
        elif op == "div" and parts[0] and not parts[1]:
            keep = parts[0]
    out_dims, used = [], set(keep)
    for d in range(nd):
        cands = []
        for i in tens:
            k = d - (nd - len(ins[i].shape))
            if k >= 0 and ins[i].shape[k] == node.shape[d] and ins[i].shape[k] > 1:
                cands.append(lays[i].dims[k])
        a = _merge_axis(cands, used)
        if a is not None:
            used.add(a)
        out_dims.append(a)
    secs = []
    for i in tens:
        for dd, sz in lays[i].sections:
            od = dd + (nd - len(ins[i].shape))
            if out_dims[od] == lays[i].dims[dd] and all(s[0] != od for s in secs):
                secs.append((od, sz))
    out = Layout(tuple(out_dims), frozenset(keep), tuple(secs))
    needs = {}
    for i in tens:
        off = nd - len(ins[i].shape)
        dims = tuple(out_dims[k + off] if ins[i].shape[k] == node.shape[k + off] and ins[i].shape[k] > 1 else None
                     for k in range(len(ins[i].shape)))
        sec = tuple((k, out.section_of(k + off)) for k in range(len(dims)) if dims[k] is not None and out.section_of(k + off))
        needs[i] = Layout(dims, lays[i].partial & keep, sec)
    return _Plan(needs, out)


def _rule_unary(node, ins, lays, mesh):
    lay = lays[0]
    if node._opname in _LINEAR_UNARY:
        return _Plan({0: lay}, lay)
    return _Plan({0: lay.resolved()}, lay.resolved())


def _rule_rowwise(node, ins, lays, mesh):
    """layer_norm / rms_norm / softmax over the last axis: that axis whole, no partial sums; gains whole."""
    x = lays[0]
    dim = (node._attrs or {}).get("dim", -1)
    dim = dim % len(x.dims)
    need = Layout(tuple(None if d == dim else a for d, a in enumerate(x.dims)), frozenset(),
                  tuple(s for s in x.sections if s[0] != dim))
    needs = {0: need}
    for i in range(1, len(ins)):
        if isinstance(ins[i], C.Tensor):
            needs[i] = lays[i].replicated()
    return _Plan(needs, need)


def _rule_linear(node, ins, lays, mesh):
    """``x[..., K] @ w[N, K]^T (+ b[N])`` (tensor/layout.go:629-714).  The activations keep their
    split; a weight dimension split over an axis the activations already use is gathered where it is
    used; a split contraction gives a partial sum; a bias joins after the sum."""
    x, w = lays[0], lays[1]
    has_bias = len(ins) > 2
    batch = list(x.dims[:-1])
    used = {a for a in batch if a is not None} | set(x.partial)
    kx, kw, nw = x.dims[-1], w.dims[1], w.dims[0]
    if nw in used:
        nw = None                                   # fully sharded weight: gathered where used
    if nw is not None:
        used.add(nw)
    k = None
    for cand in (kw, kx):                           # prefer the weight's split of the contraction
        if cand is not None and cand not in used:
            k = cand
            break
    xn = Layout(tuple(batch) + (k,), x.partial)
    nsec = w.section_of(0) if nw is not None else None
    wn = Layout((nw, k), frozenset(), ((0, nsec),) if nsec else ())
    out_partial = frozenset(x.partial | ({k} if k is not None else set()))
    nd = len(batch) + 1
    out = Layout(tuple(batch) + (nw,), out_partial, ((nd - 1, nsec),) if nsec else ())
    needs = {0: xn, 1: wn}
    if not has_bias:
        return _Plan(needs, out)
    bn = Layout((nw,), frozenset(), ((0, nsec),) if nsec else ())
    needs[2] = bn
    if not out_partial:
        return _Plan(needs, out)

    def build(loc, conv):                            # partial product, summed, then the bias (added once)
        y = C.matmul_t(loc[0], loc[1])
        y = conv(y, out, out.resolved())
        return C.add(y, loc[2])
    return _Plan(needs, out.resolved(), build)


def _rule_matmul(node, ins, lays, mesh):
    a, b = lays[0], lays[1]
    if len(ins[1].shape) != 2:
        return None
    batch = list(a.dims[:-1])
    used = {x for x in batch if x is not None} | set(a.partial)
    nb = b.dims[1] if b.dims[1] not in used else None
    if nb is not None:
        used.add(nb)
    k = None
    for cand in (b.dims[0], a.dims[-1]):
        if cand is not None and cand not in used:
            k = cand
            break
    needs = {0: Layout(tuple(batch) + (k,), a.partial), 1: Layout((k, nb))}
    return _Plan(needs, Layout(tuple(batch) + (nb,), frozenset(a.partial | ({k} if k else set()))))


def _rule_attention(node, ins, lays, mesh):
    """Attention splits over batch and heads only (tensor/layout.go:832-888)."""
    q = lays[0]
    b, h = q.dims[0], q.dims[1]
    if h is not None and any(ins[i].shape[1] % mesh.axis_size(h) for i in (1, 2)):
        h = None
    lay = Layout((b, h, None, None))
    needs = {0: lay, 1: lay, 2: lay}
    if len(ins) > 3:
        needs[3] = lays[3].replicated()
    return _Plan(needs, lay)


def _rule_reduce(node, ins, lays, mesh):
    at = node._attrs or {}
    x, op = lays[0], node._opname
    nd = len(x.dims)
    dim, keep = at.get("dim"), at.get("keepdim", False)
    red = set(range(nd)) if dim is None else {d % nd for d in ((dim,) if isinstance(dim, int) else dim)}
    if op not in ("sum", "mean"):
        need = Layout(tuple(None if d in red else a for d, a in enumerate(x.dims)))
        out = tuple(a for d, a in enumerate(need.dims) if keep or d not in red) if dim is not None else ()
        return _Plan({0: need}, Layout(out))
    split = {x.dims[d] for d in red if x.dims[d] is not None}
    out_dims = tuple((None if d in red else a) for d, a in enumerate(x.dims) if keep or d not in red) if dim is not None else ()
    out = Layout(out_dims, frozenset(x.partial | split))
    if op == "sum" or not split:
        return _Plan({0: x}, out)
    share = 1.0 / math.prod(mesh.axis_size(a) for a in split)

    fn, kw, name, at2 = node._fn, node._kw, node._opname, node._attrs

    def build(loc, conv):                            # a mean over equal blocks: the mean of the block means
        return C.mul(C._node(fn, (loc[0],), kw, name, attrs=at2), share)
    return _Plan({0: x}, out, build)


def _rule_mean_loss(node, ins, lays, mesh):
    """Elementwise losses averaged over everything: every block has the same size, so the loss is
    the sum over the ranks of (block mean / number of blocks)."""
    p = lays[0].resolved()
    needs = {i: p for i in range(len(ins)) if isinstance(ins[i], C.Tensor)}
    split = {a for a in p.dims if a is not None}
    share = 1.0 / math.prod([mesh.axis_size(a) for a in split] or [1])

    fn, kw, name = node._fn, node._kw, node._opname

    def build(loc, conv):
        return C.mul(C._node(fn, tuple(loc), kw, name), share)
    return _Plan(needs, Layout((), frozenset(split)), build if split else None)


def _rule_row_loss(node, ins, lays, mesh):
    """Losses over class scores ``[N, C, ...]``: rows may be split, the class axis is whole."""
    lg = lays[0].resolved()
    need0 = Layout((lg.dims[0], None) + tuple(lg.dims[2:]))
    need1 = Layout((need0.dims[0],) + tuple(need0.dims[2:]))
    split = {a for a in need0.dims if a is not None}
    share = 1.0 / math.prod([mesh.axis_size(a) for a in split] or [1])

    fn, kw, name = node._fn, node._kw, node._opname

    def build(loc, conv):
        return C.mul(C._node(fn, tuple(loc), kw, name), share)
    return _Plan({0: need0, 1: need1}, Layout((), frozenset(split)), build if split else None)


def _rule_gather_rows(node, ins, lays, mesh):
    """Embedding lookup: the indices keep their split, the table is whole over its rows."""
    tab, idx = lays[0], lays[1]
    used = {a for a in idx.dims if a is not None}
    c = tab.dims[1] if len(tab.dims) > 1 and tab.dims[1] not in used else None
    tn = Layout((None,) + ((c,) if len(tab.dims) > 1 else ()) + (None,) * max(0, len(tab.dims) - 2))
    return _Plan({0: tn, 1: idx.resolved()}, Layout(tuple(idx.dims) + tuple(tn.dims[1:])))


def _rule_permute(node, ins, lays, mesh):
    x = lays[0]
    at = node._attrs or {}
    nd = len(x.dims)
    if node._opname == "transpose":
        perm = list(range(nd))
        a, b = at["a"] % nd, at["b"] % nd
        perm[a], perm[b] = perm[b], perm[a]
    else:
        perm = [d % nd for d in at["dims"]]
    inv = {src: dst for dst, src in enumerate(perm)}
    return _Plan({0: x}, Layout(tuple(x.dims[p] for p in perm), x.partial, tuple((inv[d], s) for d, s in x.sections)))


def _rule_reshape(node, ins, lays, mesh):
    """A split survives a reshape when it sits on the leading dimension of a group of merged or
    divided dimensions (tensor/layout.go reshapeRule): the blocks are the same contiguous ranges."""
    x = lays[0]
    ish, osh = tuple(ins[0].shape), tuple(node.shape)
    out = [None] * len(osh)
    need = list(x.dims)
    i = j = 0
    while i < len(ish) or j < len(osh):
        i0, j0, pi, pj = i, j, 1, 1
        if i < len(ish):
            pi, i = ish[i], i + 1
        if j < len(osh):
            pj, j = osh[j], j + 1
        while pi != pj:
            if pi < pj and i < len(ish):
                pi, i = pi * ish[i], i + 1
            elif j < len(osh):
                pj, j = pj * osh[j], j + 1
            else:
                break
        for d in range(i0, i):
            a = x.dims[d]
            if a is None:
                continue
            n = mesh.axis_size(a)
            lead = next((dd for dd in range(i0, i) if ish[dd] > 1), i0)
            olead = next((dd for dd in range(j0, j) if osh[dd] > 1), j0)
            if d == lead and j0 < len(osh) and osh[olead] % n == 0 and x.section_of(d) is None and out[olead] is None:
                out[olead] = a
            else:
                need[d] = None                       # gathered before the reshape
    needl = Layout(tuple(need), x.partial)            # a sectioned dimension is gathered before a reshape
    outl = Layout(tuple(out), x.partial)
    lshape = local_shape(osh, outl, mesh)

    def build(loc, conv):
        return C.reshape(loc[0], lshape)
    return _Plan({0: needl}, outl, build)


def _rule_split(node, ins, lays, mesh):
    x = lays[0]
    at = node._attrs or {}
    d = at["dim"] % len(x.dims)
    sizes = at["sizes"]
    a = x.dims[d]
    if a is None:
        return _Plan({0: x}, x)
    sec = x.section_of(d)
    if sec is not None and isinstance(sizes, tuple) and tuple(sec) == tuple(sizes):
        n = mesh.axis_size(a)
        part = at["part"]
        lsizes = [s // n for s in sizes]
        out = Layout(x.dims, x.partial, tuple(s for s in x.sections if s[0] != d))

        def build(loc, conv):
            return C.split(loc[0], lsizes, d)[part]
        return _Plan({0: x}, out, build)
    need = Layout(tuple(None if i == d else ax for i, ax in enumerate(x.dims)), x.partial,
                  tuple(s for s in x.sections if s[0] != d))
    return _Plan({0: need}, need)


def _rule_squeeze(node, ins, lays, mesh):
    x = lays[0]
    ish, osh = tuple(ins[0].shape), tuple(node.shape)
    if node._opname == "unsqueeze":
        d = (node._attrs or {})["dim"] % len(osh)
        dims = list(x.dims)
        dims.insert(d, None)
        return _Plan({0: x}, Layout(tuple(dims), x.partial))
    dim = (node._attrs or {}).get("dim")
    drop = {d for d, sz in enumerate(ish) if sz == 1} if dim is None else ({dim % len(ish)} if ish[dim % len(ish)] == 1 else set())
    need = Layout(tuple(None if d in drop else a for d, a in enumerate(x.dims)), x.partial,
                  tuple(sc for sc in x.sections if sc[0] not in drop))
    kept = [d for d in range(len(ish)) if d not in drop]
    pos = {d: i for i, d in enumerate(kept)}
    return _Plan({0: need}, Layout(tuple(x.dims[d] for d in kept), x.partial,
                                   tuple((pos[sc[0]], sc[1]) for sc in need.sections)))


def rule_for(node, ins, lays, mesh):
    """The rules table: opname -> plan.  None means "no rule": the generic one applies (every operand
    whole, the op runs replicated), as in the reference."""
    op = node._opname
    if op in _BINARY:
        return _rule_elementwise(node, ins, lays, mesh)
    if op in _LINEAR_UNARY or op in _NONLINEAR_UNARY:
        return _rule_unary(node, ins, lays, mesh)
    if op in ("layer_norm", "rms_norm", "softmax", "log_softmax"):
        return _rule_rowwise(node, ins, lays, mesh)
    if op == "linear":
        return _rule_linear(node, ins, lays, mesh)
    if op == "matmul":
        return _rule_matmul(node, ins, lays, mesh)
    if op == "attention":
        return _rule_attention(node, ins, lays, mesh)
    if op in ("sum", "mean", "max", "min", "var", "logsumexp"):
        return _rule_reduce(node, ins, lays, mesh)
    if op in _MEAN_LOSSES:
        return _rule_mean_loss(node, ins, lays, mesh)
    if op in _ROW_LOSSES:
        return _rule_row_loss(node, ins, lays, mesh)
    if op == "gather_rows":
        return _rule_gather_rows(node, ins, lays, mesh)
    if op in ("permute", "transpose"):
        return _rule_permute(node, ins, lays, mesh)
    if op == "reshape":
        return _rule_reshape(node, ins, lays, mesh)
    if op == "split":
        return _rule_split(node, ins, lays, mesh)
    if op in ("squeeze", "unsqueeze"):
        return _rule_squeeze(node, ins, lays, mesh)
    return None


def _generic(node, ins, lays):
    needs = {i: lays[i].replicated() for i, a in enumerate(ins) if isinstance(a, C.Tensor)}
    return _Plan(needs, Layout((None,) * len(node.shape)))


# =========================================================================== analyse + lower
_ANALYSES: dict = {}
_STATS = {"analysed": 0, "reused": 0}


def stats() -> dict:
    return dict(_STATS, cached=len(_ANALYSES))


def _walk(roots):
    order, seen, leaves = [], set(), []
    for root in roots:
        stack = [(root, False)]
        while stack:
            t, done = stack.pop()
            if id(t) in seen:
                continue
            if isinstance(t, MeshTensor) or t._fn is None or t._val is not None:
                seen.add(id(t))
                leaves.append(t)
                continue
            if done:
                seen.add(id(t))
                order.append(t)
                continue
            stack.append((t, True))
            for a in reversed([a for a in C._flatten(t._args) if isinstance(a, C.Tensor)]):
                if id(a) not in seen:
                    stack.append((a, False))
    return order, leaves


def _flat_inputs(t):
    return [a for a in C._flatten(t._args)]


def _structure_key(order, leaves, roots, mesh):
    idx = {}
    for i, t in enumerate(leaves):
        idx[id(t)] = ("l", i)
    for i, t in enumerate(order):
        idx[id(t)] = ("n", i)
    parts = [("mesh", mesh.shape, mesh.axes)]
    for t in leaves:
        lay = t.layout if isinstance(t, MeshTensor) else None
        parts.append((tuple(t.shape), t.dtype, lay))
    try:
        for t in order:
            at = tuple(sorted((k, v if not isinstance(v, list) else tuple(v)) for k, v in (t._attrs or {}).items()))
            parts.append((t._opname, at, tuple(t.shape), tuple(idx[id(a)] if isinstance(a, C.Tensor) else repr(a)
                                                              for a in _flat_inputs(t))))
        parts.append(tuple(idx[id(r)] for r in roots))
        key = tuple(parts)
        hash(key)
        return key
    except TypeError:
        return None


def analyse(roots, mesh: Mesh):
    """Layouts for every node below ``roots``: ``({id(node): plan}, order, leaves, depth)``; cached by
    structure.  ``depth`` is the number of collectives on the longest path (tensor/partition.go:41-81)."""
    order, leaves = _walk(roots)
    key = _structure_key(order, leaves, roots, mesh)
    cached = _ANALYSES.get(key) if key is not None else None
    lay = {}
    for t in leaves:
        lay[id(t)] = t.layout if isinstance(t, MeshTensor) else Layout((None,) * len(t.shape))
    if cached is not None:
        _STATS["reused"] += 1
        plans = {id(t): p for t, p in zip(order, cached)}
        return plans, order, leaves
    plans = {}
    for t in order:
        ins = _flat_inputs(t)
        lays = [lay.get(id(a)) if isinstance(a, C.Tensor) else None for a in ins]
        plan = None
        try:
            plan = rule_for(t, ins, lays, mesh)
        except (KeyError, IndexError, TypeError):
            plan = None
        if plan is None:
            plan = _generic(t, ins, lays)
        plans[id(t)] = plan
        lay[id(t)] = plan.out
    _STATS["analysed"] += 1
    if key is not None:
        if len(_ANALYSES) > 64:
            _ANALYSES.clear()
        _ANALYSES[key] = [plans[id(t)] for t in order]
    return plans, order, leaves


def lower(roots, mesh: Mesh, want=None):
    """This rank's graph of ``roots``: local lazy tensors in the layouts ``want`` (default: whole)."""
    plans, order, leaves = analyse(roots, mesh)
    local, lay, conv_cache = {}, {}, {}
    for t in leaves:
        if isinstance(t, MeshTensor):
            leaf = C.from_torch(t.local)
            if t.param is not None:
                leaf._stale = (t.param, t.param._version)
            local[id(t)], lay[id(t)] = leaf, t.layout
        else:
            local[id(t)], lay[id(t)] = t, Layout((None,) * len(t.shape))

    def conv_of(node_id, x, src, dst, marks=frozenset()):
        if src == dst and not marks:
            return x
        k = (node_id, dst, frozenset(marks))
        if k not in conv_cache:
            conv_cache[k] = convert(x, src, dst, mesh, marks)
        return conv_cache[k]

    # Where must a cotangent be summed over a mesh axis?  A value that is whole over axis a and meets
    # an op whose result is split over a gets a partial cotangent from it.  The sum may move down
    # through a producer with a single differentiable operand that is whole over a as well (the
    # producer's Jacobian is then the same on every rank of a), provided every reader of the value
    # wants it; at a sharded parameter it fuses with the all-gather into gather / reduce-scatter.
    sums, pushed = {}, {}
    uses = {}
    for t in order:
        for i, a in enumerate(_flat_inputs(t)):
            if isinstance(a, C.Tensor):
                uses.setdefault(id(a), []).append((id(t), i))
    for t in reversed(order):
        plan = plans[id(t)]
        ins = _flat_inputs(t)
        readers = uses.get(id(t), [])
        common = set.intersection(*[set(sums.get(u, ())) for u in readers]) if readers else set()
        floats = [i for i, a in enumerate(ins) if isinstance(a, C.Tensor) and a.dtype.is_floating_point]
        can = set()
        if plan.build is None and len(floats) == 1 and id(t) not in {id(r) for r in roots}:
            need = plan.needs.get(floats[0], lay.get(id(ins[floats[0]])))
            can = {a for a in common if a not in plan.out.axes() and (need is None or a not in need.axes())}
        pushed[id(t)] = can
        out_axes = {a for a in plan.out.dims if a is not None} | can
        for i in floats:
            need = plan.needs.get(i)
            used = need.axes() if need is not None else set()
            sums[(id(t), i)] = frozenset(ax for ax in out_axes if ax not in used)

    for t in order:
        plan = plans[id(t)]
        ins = _flat_inputs(t)
        loc = []
        for i, a in enumerate(ins):
            if not isinstance(a, C.Tensor):
                loc.append(a)
                continue
            need = plan.needs.get(i, lay[id(a)])
            marks = frozenset(sums.get((id(t), i), frozenset()) - pushed.get(id(a), set()))
            loc.append(conv_of(id(a), local[id(a)], lay[id(a)], need, marks))
        if plan.build is not None:
            tl = [x for x in loc if isinstance(x, C.Tensor)]
            node = plan.build(tl, lambda y, s, d: convert(y, s, d, mesh))
        else:
            node = C._node(t._fn, _rebuild_args(t._args, iter(loc)), t._kw, t._opname, attrs=t._attrs)
        if isinstance(node, C.Tensor) and node._err is not None:
            raise node._err
        local[id(t)], lay[id(t)] = node, plan.out
    outs = []
    for i, r in enumerate(roots):
        dst = (want[i] if want is not None and want[i] is not None else lay[id(r)].replicated())
        outs.append(conv_of(id(r), local[id(r)], lay[id(r)], dst))
    return outs


def _rebuild_args(args, it):
    out = []
    for a in args:
        if isinstance(a, (list, tuple)):
            out.append(type(a)(_rebuild_args(a, it)))
        else:
            out.append(next(it))
    return tuple(out)


# =========================================================================== public entry points
def on_mesh(t: C.Tensor):
    """The mesh a lazy tensor's graph lives on, or None."""
    sh = getattr(t, "_sharding", None)
    return sh[0] if sh else None


def _find_mesh(roots):
    _, leaves = _walk(roots)
    for t in leaves:
        if isinstance(t, MeshTensor):
            return t.mesh
    return None


def realize_blocks(*tensors: C.Tensor):
    """Computes sharded lazy tensors and leaves every result where the rules put it: returns
    ``[(local torch tensor, Layout)]`` without gathering anything (partial sums are completed)."""
    mesh = _find_mesh(tensors)
    plans, order, leaves = analyse(list(tensors), mesh)
    lays = []
    for t in tensors:
        if id(t) in plans:
            lays.append(plans[id(t)].out.resolved())
        else:
            lays.append(t.layout if isinstance(t, MeshTensor) else Layout((None,) * len(t.shape)))
    outs = lower(list(tensors), mesh, want=lays)
    C.realize(*outs)
    return [(o._val, l) for o, l in zip(outs, lays)]


def realize(*tensors: C.Tensor) -> None:
    """Computes sharded lazy tensors; each becomes a realized tensor holding the WHOLE value (what a
    single device would hold), gathered from the ranks."""
    todo = [t for t in tensors if t._val is None and not isinstance(t, MeshTensor)]
    for t in tensors:
        if isinstance(t, MeshTensor) and t._val is None:      # a leaf: gather its blocks
            (o,) = lower([t], t.mesh)
            C.realize(o)
            t._assign(o._val)
    if not todo:
        return
    mesh = _find_mesh(todo)
    outs = lower(todo, mesh)
    C.realize(*outs)
    for t, o in zip(todo, outs):
        t._assign(o._val)
        t._fn, t._args, t._kw = None, (), {}
        t._sharding = None


def backward(loss: C.Tensor) -> None:
    """Loss and every parameter gradient of a sharded graph in one pass; each gradient arrives in
    the layout of its parameter (the collectives that takes are part of the backward pass)."""
    mesh = _find_mesh([loss])
    (local_loss,) = lower([loss], mesh)
    from ..tensor.autograd import backward as plain_backward
    plain_backward(local_loss)
    loss._assign(local_loss._val)
    loss._fn, loss._args, loss._kw = None, (), {}
    loss._sharding = None


def sharded_step(model, opt, mesh: Mesh, loss_fn, x, y, data_axis: str = "data") -> float:
    """One training step on a batch that every rank passes whole: the batch is placed ``P(data)``,
    the graph is partitioned, the optimizer updates the local blocks (no collective: states are
    laid out like the parameters)."""
    spec_x = PartitionSpec((data_axis,)) if data_axis in mesh.axes and mesh.axis_size(data_axis) > 1 else None
    xs = place(x, mesh, spec_x)
    ys = place(y, mesh, spec_x) if y is not None else None
    loss = loss_fn(model(xs), ys)
    backward(loss)
    opt.step()
    opt.zero_grad()
    return float(loss.item())
