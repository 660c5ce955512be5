"""Device meshes and sharded training, SPMD style: one process per device.

The reference partitions ONE lazy graph over the devices of one process
(tensor/mesh.go, layout.go, partition.go, reshard.go).  Here every rank runs the
same program on its shard and the layout rules show up as the collectives that
sharded layers insert:

* column-parallel product (weight split by output rows): no collective forward,
  all-reduce of the input gradient backward;
* row-parallel product (weight split by input columns): partial sums -> one
  all-reduce forward (tensor/layout.go:832-888), none backward;
* fully sharded weight (ZeRO-3, nn/shard.go:74-89): all-gather where used,
  reduce-scatter of its gradient; the gathered copy made by forward is reused by
  backward of the same step (no second gather, train/sharded_test.go:198-274);
* data axis: gradients become partial over "data" -> all-reduce (or the
  reduce-scatter above when the weight is sharded over the same axis).

``Mesh.traffic`` counts collectives and bytes per kind like ``Mesh.Traffic``
(tensor/mesh.go:66-96).  Collectives here and in the per-op partitioner
(``parallel/spmd.py``, which ``fit(sharded=...)`` uses) are ``torch.distributed``
calls on process groups (NCCL on GPUs, gloo on CPU ranks for tests).  The fused
all-gather + product and product + reduce-scatter kernels of
``parallel/fused_gemm.py`` are called by the Llama engines (``models/llama.py``), not
by these wrappers.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .. import tensor as T
from ..tensor.autograd import Param


@dataclass
class Traffic:
    all_reduce: int = 0
    all_gather: int = 0
    reduce_scatter: int = 0
    broadcast: int = 0
    bytes: int = 0

    def reset(self):
        self.all_reduce = self.all_gather = self.reduce_scatter = self.broadcast = self.bytes = 0

    def total(self) -> int:
        return self.all_reduce + self.all_gather + self.reduce_scatter + self.broadcast


class PartitionSpec(tuple):
    """Axis name (or None) per tensor dimension; ``with_sections`` splits a fused dimension
    (e.g. [Q | K | V] rows) section by section (tensor/mesh.go:270-281)."""

    sections = None

    def with_sections(self, dim: int, *sizes: int) -> "PartitionSpec":
        p = PartitionSpec(self)
        p.sections = (dim, tuple(sizes))
        return p


def P(*axes) -> PartitionSpec:
    return PartitionSpec(axes)


class Mesh:
    """An n-dimensional grid of ranks (row-major), at most 8 axes (tensor/mesh.go:99)."""

    def __init__(self, shape, axes, ranks=None):
        shape, axes = tuple(shape), tuple(axes)
        if len(shape) != len(axes) or len(shape) > 8:
            raise T.ErrShape("mesh shape and axis names must have the same length (at most 8)")
        self.shape, self.axes = shape, axes
        self.size = math.prod(shape)
        world = dist.get_world_size() if dist.is_initialized() else 1
        self.ranks = list(ranks) if ranks is not None else list(range(self.size))
        if self.size != len(self.ranks) or self.size > world:
            raise T.ErrShape(f"mesh of {self.size} devices does not fit {world} ranks")
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.traffic = Traffic()
        self._groups = {}
        me = self.ranks.index(self.rank) if self.rank in self.ranks else 0
        self.coords = {}
        rem = me
        for ax, n in zip(reversed(axes), reversed(shape)):
            self.coords[ax] = rem % n
            rem //= n
        # every rank creates every sub-group in the same order (a torch.distributed requirement)
        for ax in axes:
            self._make_groups(ax)

    def _make_groups(self, axis: str):
        i = self.axes.index(axis)
        n = self.shape[i]
        stride = math.prod(self.shape[i + 1:])
        mine = None
        seen = set()
        for base in range(self.size):
            if base in seen:
                continue
            coord = (base // stride) % n
            if coord != 0:
                continue
            members = [base + k * stride for k in range(n)]
            seen.update(members)
            ranks = [self.ranks[m] for m in members]
            g = dist.new_group(ranks) if (dist.is_initialized() and n > 1 and self.size > 1) else None
            if self.rank in ranks:
                mine = (g, ranks)
        self._groups[axis] = mine or (None, [self.rank])

    def axis_size(self, axis: str) -> int:
        return self.shape[self.axes.index(axis)]

    def axis_index(self, axis: str) -> int:
        return self.coords[axis]

    def group(self, axis: str):
        return self._groups[axis][0]

    def close(self):
        for g, _ in self._groups.values():
            if g is not None:
                dist.destroy_process_group(g)
        self._groups = {}

    # ---------------------------------------------------------- collectives
    def _count(self, kind: str, t: torch.Tensor):
        setattr(self.traffic, kind, getattr(self.traffic, kind) + 1)
        self.traffic.bytes += t.numel() * t.element_size()

    def all_reduce(self, t: torch.Tensor, axis: str, op="sum") -> torch.Tensor:
        if self.axis_size(axis) == 1:
            return t
        self._count("all_reduce", t)
        out = t.clone()
        dist.all_reduce(out, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM, group=self.group(axis))
        return out

    def all_gather(self, t: torch.Tensor, axis: str, dim: int = 0) -> torch.Tensor:
        n = self.axis_size(axis)
        if n == 1:
            return t
        self._count("all_gather", t)
        parts = [torch.empty_like(t) for _ in range(n)]
        dist.all_gather(parts, t.contiguous(), group=self.group(axis))
        return torch.cat(parts, dim)

    def reduce_scatter(self, t: torch.Tensor, axis: str, dim: int = 0) -> torch.Tensor:
        n = self.axis_size(axis)
        if n == 1:
            return t
        self._count("reduce_scatter", t)
        chunks = [c.contiguous() for c in t.chunk(n, dim)]
        out = torch.empty_like(chunks[0])
        if t.device.type == "cpu":  # gloo has no reduce_scatter: all-reduce and cut (same result)
            full = t.clone()
            dist.all_reduce(full, group=self.group(axis))
            return full.chunk(n, dim)[self.axis_index(axis)].contiguous()
        dist.reduce_scatter(out, chunks, group=self.group(axis))
        return out

    def local_slice(self, t: torch.Tensor, spec: PartitionSpec) -> torch.Tensor:
        """This rank's block of a replicated tensor under ``spec`` (splits must be even)."""
        for d, ax in enumerate(spec):
            if ax is None:
                continue
            n, i = self.axis_size(ax), self.axis_index(ax)
            sec = spec.sections
            if sec is not None and sec[0] == d:
                parts, off = [], 0
                for size in sec[1]:
                    if size % n:
                        raise T.ErrShape(f"section of {size} rows does not split {n} ways")
                    per = size // n
                    parts.append(t.narrow(d, off + i * per, per))
                    off += size
                t = torch.cat(parts, d)
            else:
                if t.shape[d] % n:
                    raise T.ErrShape(f"dimension {d} of size {t.shape[d]} does not split {n} ways")
                per = t.shape[d] // n
                t = t.narrow(d, i * per, per)
        return t.contiguous()


# ---------------------------------------------------------------------------
# differentiable collectives
# ---------------------------------------------------------------------------
class _CopyToAxis(torch.autograd.Function):
    """Identity forward, all-reduce of the gradient backward (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, mesh, axis):
        ctx.mesh, ctx.axis = mesh, axis
        return x

    @staticmethod
    def backward(ctx, g):
        return ctx.mesh.all_reduce(g, ctx.axis), None, None


class _ReduceFromAxis(torch.autograd.Function):
    """All-reduce forward (partial sums of a row-parallel layer), identity backward."""

    @staticmethod
    def forward(ctx, x, mesh, axis):
        return mesh.all_reduce(x, axis)

    @staticmethod
    def backward(ctx, g):
        return g, None, None


class _GatherWeight(torch.autograd.Function):
    """All-gather of a sharded weight where it is used; its gradient is reduce-scattered
    back to the shard layout.  The gathered copy is cached on the module for the step."""

    @staticmethod
    def forward(ctx, shard, mesh, axis, dim):
        ctx.mesh, ctx.axis, ctx.dim = mesh, axis, dim
        return mesh.all_gather(shard, axis, dim)

    @staticmethod
    def backward(ctx, g):
        return ctx.mesh.reduce_scatter(g.contiguous(), ctx.axis, ctx.dim), None, None, None


class _GradAllReduce(torch.autograd.Function):
    """Identity forward; the gradient (partial over the data axis) is all-reduced."""

    @staticmethod
    def forward(ctx, w, mesh, axis):
        ctx.mesh, ctx.axis = mesh, axis
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        return ctx.mesh.all_reduce(g, ctx.axis), None, None


def copy_to(x: T.Tensor, mesh: Mesh, axis: str) -> T.Tensor:
    return T.core._node(lambda v: v if v.device.type == "meta" else _CopyToAxis.apply(v, mesh, axis), (x,), {}, "copy_to_axis")


def reduce_from(x: T.Tensor, mesh: Mesh, axis: str) -> T.Tensor:
    return T.core._node(lambda v: v if v.device.type == "meta" else _ReduceFromAxis.apply(v, mesh, axis), (x,), {}, "all_reduce")


# ---------------------------------------------------------------------------
# sharding rules for modules (nn.Shard / Rules / FullyShard / TensorParallel)
# ---------------------------------------------------------------------------
@dataclass
class ShardRule:
    """``match(name, param) -> PartitionSpec or None``."""
    match: object
    name: str = "rule"


def _is_2d_weight(name, p):
    return p._data.dim() >= 2


def fully_shard(axis: str = "data") -> ShardRule:
    """Split the first evenly divisible axis of every parameter over ``axis`` (nn.FullyShard)."""
    def match(name, p, mesh):
        n = mesh.axis_size(axis)
        for d, s in enumerate(p.shape):
            if s % n == 0 and s >= n:
                return P(*([None] * d + [axis] + [None] * (len(p.shape) - d - 1)))
        return None
    return ShardRule(match, "fully_shard")


def tensor_parallel(axis: str = "model") -> ShardRule:
    """Megatron split (nn.TensorParallel, nn/shard.go:102-158): up/gate and fused QKV by output
    rows (QKV section by section), down and attention-out by input columns."""
    def match(name, p, mesh):
        leaf = name.split(".")
        if len(leaf) < 2:
            return None
        layer, kind = leaf[-2], leaf[-1]
        if layer in ("up", "gate", "qkv", "q", "k", "v", "fc"):
            return P(axis, None) if kind == "weight" else P(axis)
        if layer in ("down", "out", "proj", "o") and kind == "weight":
            return P(None, axis)
        return None
    return ShardRule(match, "tensor_parallel")


def rules(*rs: ShardRule) -> ShardRule:
    """First matching rule wins (nn.Rules)."""
    def match(name, p, mesh):
        for r in rs:
            spec = r.match(name, p, mesh)
            if spec is not None:
                return spec
        return None
    return ShardRule(match, "rules")


def shard_module(model, mesh: Mesh, rule: ShardRule | None, data_axis: str = "data"):
    """Shards ``model`` in place over ``mesh``: parameters keep only their local block, layers
    gain the collectives their layout needs.  With ``rule=None`` parameters stay replicated and
    only gradients are all-reduced over the data axis (``train.Sharded(mesh, nil)``)."""
    from ..nn.module import Linear
    from ..nn.transformer import SelfAttention
    named = dict(model.named_params())
    specs = {}
    for name, p in named.items():
        spec = rule.match(name, p, mesh) if rule is not None else None
        specs[name] = spec
    # attach layouts
    for name, p in named.items():
        spec = specs[name]
        p._mesh = mesh
        p._spec = spec
        if spec is not None:
            full = p._data
            secs = None
            owner = _owner_module(model, name)
            if isinstance(owner, Linear) and getattr(owner, "_qkv_sections", None) and spec[0] is not None \
                    and spec[0] != data_axis:  # only a head split needs sections; a fully sharded weight is cut plainly
                spec = spec.with_sections(0, *owner._qkv_sections)
                p._spec = spec
            p._full_shape = tuple(full.shape)
            p._data = mesh.local_slice(full, spec).clone()
            p._version += 1
            if data_axis in spec:
                p._gather = _make_gather(mesh, data_axis, list(spec).index(data_axis), p)
    for m in model.modules():
        if isinstance(m, SelfAttention):
            _shard_attention(m, mesh, data_axis)
    for m in model.modules():
        if isinstance(m, Linear):
            _wrap_linear(m, mesh, data_axis)
    model._mesh = mesh
    return model


def _make_gather(mesh, axis, dim, p):
    def gather(leaf):
        def run(v):
            if v.device.type == "meta":
                shape = list(v.shape)
                shape[dim] *= mesh.axis_size(axis)
                return torch.empty(shape, dtype=v.dtype, device="meta")
            return _GatherWeight.apply(v, mesh, axis, dim)
        return T.core._node(run, (leaf,), {}, "all_gather")
    return gather


def _owner_module(model, pname):
    obj = model
    for part in pname.split(".")[:-1]:
        if part.isdigit():
            obj = obj[int(part)] if isinstance(obj, (list, tuple)) else obj
        else:
            nxt = getattr(obj, part, None)
            obj = nxt if nxt is not None else obj
        if isinstance(obj, list):
            continue
    return obj


def _shard_attention(att, mesh, data_axis):
    """Heads split over the model axis that shards the fused QKV rows (attention splits over heads
    only); a weight that is merely fully sharded over the data axis is gathered whole, heads stay."""
    spec = getattr(att.qkv.weight, "_spec", None)
    if spec is None or spec[0] is None or spec[0] == data_axis:
        return
    n = mesh.axis_size(spec[0])
    if att.heads % n or att.kv_heads % n:
        raise T.ErrShape("attention heads do not divide by the tensor-parallel size")
    att.heads //= n
    att.kv_heads //= n


def _wrap_linear(lin, mesh: Mesh, data_axis: str):
    """Tensor-parallel products.  (Weights sharded over the data axis arrive gathered through
    ``Param.value``, so they look replicated here.)"""
    w_spec = getattr(lin.weight, "_spec", None)
    ax0 = w_spec[0] if w_spec is not None and w_spec[0] != data_axis else None
    ax1 = w_spec[1] if w_spec is not None and len(w_spec) > 1 and w_spec[1] != data_axis else None
    if ax0 is None and ax1 is None:
        return

    def forward(x):
        w = lin.weight.value()
        b = lin.bias.value() if lin.bias is not None else None
        args = (x, w) + ((b,) if b is not None else ())

        def run(v, wt, *bb):
            if v.device.type == "meta":
                return torch.empty(*v.shape[:-1], wt.shape[0], dtype=v.dtype, device="meta")
            bias = bb[0] if bb else None
            if ax0 is not None:  # column parallel: output stays split, input gradient is all-reduced
                return torch.nn.functional.linear(_CopyToAxis.apply(v, mesh, ax0), wt, bias)
            # row parallel: partial sums, one all-reduce, bias added once afterwards
            y = _ReduceFromAxis.apply(torch.nn.functional.linear(v, wt), mesh, ax1)
            return y + bias if bias is not None else y
        return T.core._node(run, args, {}, "sharded_linear")
    lin.forward = forward


def gather_param(p: Param) -> torch.Tensor:
    """The whole value of a (possibly sharded) parameter, for tests and checkpoints."""
    mesh, spec = getattr(p, "_mesh", None), getattr(p, "_spec", None)
    if mesh is None or spec is None:
        return p._data
    t = p._data
    for d, ax in enumerate(spec):
        if ax is None:
            continue
        n = mesh.axis_size(ax)
        parts = [torch.empty_like(t) for _ in range(n)]
        if n > 1:
            dist.all_gather(parts, t.contiguous(), group=mesh.group(ax))
        else:
            parts = [t]
        sec = spec.sections
        if sec is not None and sec[0] == d:
            pieces, off = [], 0
            for size in sec[1]:
                per = size // n
                pieces.append(torch.cat([pp.narrow(d, off, per) for pp in parts], d))
                off += per
            t = torch.cat(pieces, d)
        else:
            t = torch.cat(parts, d)
    return t


def reduce_gradients(model, mesh: Mesh, data_axis: str = "data") -> None:
    """The step's collectives: every gradient that is still partial over the data axis
    (parameters not sharded over it) is all-reduced (tensor/layout.go:629-714)."""
    if data_axis not in mesh.axes or mesh.axis_size(data_axis) == 1:
        return
    for _, p in model.named_params(buffers=False):
        if p._grad is None:
            continue
        spec = getattr(p, "_spec", None)
        if spec is not None and data_axis in spec:
            continue  # reduce-scattered by the gather's backward already
        p._grad = mesh.all_reduce(p._grad, data_axis)


def sharded_step(model, opt, mesh: Mesh, loss_fn, x, y, data_axis: str = "data") -> float:
    """One training step on this rank's share of the batch; returns the global mean loss."""
    dp = mesh.axis_size(data_axis) if data_axis in mesh.axes else 1
    loss = loss_fn(model(x), y) * (1.0 / dp)
    loss.backward()
    reduce_gradients(model, mesh, data_axis)
    opt.step()
    opt.zero_grad()
    total = torch.tensor([loss.item()], dtype=torch.float64)
    if dp > 1:
        total = mesh.all_reduce(total, data_axis)
    return float(total[0])


# ---------------------------------------------------------------------------
# tensors with a sharding (tensor.Shard / WithSharding / Tensor.Sharding, tensor/mesh.go:218-314)
# ---------------------------------------------------------------------------
def shard(x: T.Tensor, mesh: Mesh, spec: PartitionSpec) -> T.Tensor:
    """This rank's block of a replicated tensor under ``spec``; the result remembers its sharding."""
    out = T.from_torch(mesh.local_slice(x.data(), spec))
    out._sharding = (mesh, spec)
    return out


def sharding_of(x: T.Tensor):
    """``(mesh, spec)`` of a tensor made by ``shard`` / ``with_sharding``, else None (replicated)."""
    return getattr(x, "_sharding", None)


def unshard(x: T.Tensor) -> T.Tensor:
    """The whole tensor on every rank: one all-gather per split dimension (sections regrouped)."""
    sh = sharding_of(x)
    if sh is None:
        return x
    mesh, spec = sh
    v = x.data()
    for d, ax in enumerate(spec):
        if ax is None or mesh.axis_size(ax) == 1:
            continue
        n = mesh.axis_size(ax)
        full = mesh.all_gather(v, ax, d)
        sec = spec.sections
        if sec is not None and sec[0] == d:
            # gathered order is [rank][section]; the tensor's own order is [section][rank]
            per = [s // n for s in sec[1]]
            blocks = full.split([p for _ in range(n) for p in per], d)
            order = [blocks[r * len(per) + s] for s in range(len(per)) for r in range(n)]
            full = torch.cat(order, d)
        v = full
    return T.from_torch(v)


def with_sharding(x: T.Tensor, mesh: Mesh, spec: PartitionSpec) -> T.Tensor:
    """Converts ``x`` to the layout ``spec``.  There is no all-to-all: a split that moves from one axis
    to another is gathered and cut again, as in the reference."""
    cur = sharding_of(x)
    if cur is not None and cur[0] is mesh and tuple(cur[1]) == tuple(spec) and cur[1].sections == spec.sections:
        return x
    return shard(unshard(x), mesh, spec)
