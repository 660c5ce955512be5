"""Parameters, reverse-mode differentiation and function transforms.

``Param`` is the only mutable object (tensor/autograd.go:830-1020): optimizers
write new values in place, after which tensors obtained from ``value()`` before
the write are stale (``ErrOverwritten``).  ``backward(loss)`` evaluates the loss
and all gradients in ONE pass and accumulates into existing gradients
(tensor/autograd.go:322-345); the differentiation itself is PyTorch autograd
over the executed graph.  ``grad / vjp / jvp / jacobian / hessian / vmap`` wrap
``torch.func`` around functions written against the lazy ``Tensor`` API
(tensor/transform.go, tensor/vmap.go).
"""
from __future__ import annotations

import weakref

import torch

from . import core as C
from . import errors as E


class Param:
    """A trainable (or frozen) tensor with an accumulated gradient."""

    def __init__(self, value, name: str = "", trainable: bool = True):
        v = value.data() if isinstance(value, C.Tensor) else torch.as_tensor(value)
        self._data = v.detach().clone()
        self._grad = None
        self._grad_buf = None       # persistent gradient storage when an optimizer keeps flat buffers
        self._version = 0
        self.name = name
        self._trainable = trainable
        self._sharding = None

    # -- value access
    def value(self) -> C.Tensor:
        if getattr(self, "_spmd", None) is not None:
            # a parameter with a layout on a device mesh: graphs built from it are partitioned
            from ..parallel.spmd import _param_leaf
            return _param_leaf(self)
        t = C.from_torch(self._data)
        t._stale = (self, self._version)
        t._fn = None
        _LEAF_PARAM[id(t)] = self
        gather = getattr(self, "_gather", None)
        if gather is not None:
            # a fully sharded parameter is all-gathered where it is used; the gradient of the
            # gathered value is reduce-scattered back onto the shard (nn/shard.go:74-89)
            return gather(t)
        return t

    def _raw(self) -> torch.Tensor:
        """The storage as it is, without computing a pending recipe (see ``Buffer``)."""
        return self._data

    def grad(self):
        return None if self._grad is None else C.from_torch(self._grad)

    def zero_grad(self) -> None:
        self._grad = None

    def set(self, value) -> None:
        v = value.data() if isinstance(value, C.Tensor) else torch.as_tensor(value)
        if tuple(v.shape) != tuple(self._data.shape):
            raise E.ErrShape(f"Param.set: shape {tuple(v.shape)} != {tuple(self._data.shape)}")
        self._data.copy_(v.to(self._data.dtype))
        self._version += 1

    def to(self, device: C.Device) -> "Param":
        self._data = self._data.to(device.torch)
        if self._grad is not None:
            self._grad = self._grad.to(device.torch)
        self._grad_buf = None
        self._version += 1
        return self

    def cast(self, dtype) -> "Param":
        self._data = self._data.to(dtype)
        self._grad = None
        self._grad_buf = None
        self._version += 1
        return self

    def freeze(self) -> "Param":
        self._trainable = False
        return self

    def unfreeze(self) -> "Param":
        self._trainable = True
        return self

    @property
    def frozen(self) -> bool:
        return not self._trainable

    @property
    def trainable(self) -> bool:
        return self._trainable

    @property
    def shape(self):
        return tuple(self._data.shape)

    @property
    def dtype(self):
        return self._data.dtype

    @property
    def device(self) -> C.Device:
        return C._dev_of(self._data)

    def shard(self, mesh, spec) -> "Param":
        self._sharding = (mesh, spec)
        return self

    def numel(self) -> int:
        return self._data.numel()


class Buffer(Param):
    """Non-trainable state (running statistics, caches): ``NewBuffer`` in the reference.

    ``set`` accepts a lazy tensor (tensor/autograd.go:929-950): the buffer then holds the recipe and
    takes the value when it is next read, when a backward pass computes it as an effect, or before
    any parameter is written in place (``flush_lazy``), so the recipe never reads overwritten
    memory."""

    def __init__(self, value, name: str = ""):
        self.__dict__["_lazy"] = None
        super().__init__(value, name, trainable=False)

    @property
    def _data(self):
        lazy = self.__dict__.get("_lazy")
        if lazy is not None:
            self.__dict__["_lazy"] = None
            _LAZY.discard(self)
            buf = self.__dict__["_buf"]
            buf.copy_(lazy.data().to(buf.dtype))
            self._version += 1
        return self.__dict__["_buf"]

    @_data.setter
    def _data(self, v):
        self.__dict__["_lazy"] = None
        self.__dict__["_buf"] = v

    def _raw(self) -> torch.Tensor:
        return self.__dict__["_buf"]

    def set(self, value) -> None:
        if isinstance(value, C.Tensor) and value._err is None and value._val is None:
            if tuple(value.shape) != tuple(self.__dict__["_buf"].shape):
                raise E.ErrShape(f"Param.set: shape {tuple(value.shape)} != {tuple(self.__dict__['_buf'].shape)}")
            self._data  # noqa: B018 - an older recipe is computed before it is replaced
            self.__dict__["_lazy"] = value
            _LAZY.add(self)
            return
        super().set(value)


_LAZY = weakref.WeakSet()


def flush_lazy() -> None:
    """Computes every buffer that still holds a recipe; called before parameters are written in
    place, so that a recipe never reads memory a step has overwritten."""
    for b in list(_LAZY):
        b._data  # noqa: B018


_LEAF_PARAM = weakref.WeakValueDictionary()


def _collect_params(root: C.Tensor) -> dict:
    """Leaf tensors below ``root`` that view parameter storage: id(leaf) -> Param."""
    out, seen, stack = {}, set(), [root]
    while stack:
        t = stack.pop()
        if id(t) in seen:
            continue
        seen.add(id(t))
        if t._stale is not None:
            out[id(t)] = (t, t._stale[0])
        stack.extend(a for a in C._flatten(t._args) if isinstance(a, C.Tensor))
    return out


def _collect_effects(root: C.Tensor) -> list:
    out, seen, stack = [], set(), [root]
    while stack:
        t = stack.pop()
        if id(t) in seen:
            continue
        seen.add(id(t))
        for e in t._effects:
            if isinstance(e, C.Tensor) and e._val is None and all(e is not o for o in out):
                out.append(e)
        stack.extend(a for a in C._flatten(t._args) if isinstance(a, C.Tensor))
    return out


def backward(loss: C.Tensor, effects=()) -> None:
    """Loss, all parameter gradients and the effects the loss carries (``with_effects``) in one pass;
    gradients accumulate in place."""
    if loss._err is not None:
        raise loss._err
    if loss.numel() != 1:
        raise E.ErrShape(f"backward needs a scalar loss, got shape {loss.shape}")
    if loss._fn is None:
        raise E.ErrNoGrad("the loss does not depend on any recorded operation")
    if C._on_mesh(loss):
        from ..parallel import spmd
        return spmd.backward(loss)
    leaves = _collect_params(loss)
    trainable = {k: (t, p) for k, (t, p) in leaves.items() if p._trainable}
    if not trainable:
        raise E.ErrNoGrad("the loss depends on no trainable parameter")
    carried = _collect_effects(loss)
    for e in carried:
        for k, v in _collect_params(e).items():
            leaves.setdefault(k, v)
    from .memory import reserve
    reserve([loss])
    memo, inputs = {}, {}
    for k, (t, p) in leaves.items():
        C._check_leaf(t)
        v = p._raw().detach()
        if p._trainable:
            if not v.dtype.is_floating_point:
                raise E.ErrNotDifferentiable(f"parameter {p.name!r} has dtype {v.dtype}")
            v = inputs.setdefault(id(p), v.requires_grad_(True))
        memo[k] = v
    with torch.enable_grad():
        out, *side = C.evaluate([loss] + carried, memo, reuse_cached=False)
        if not out.requires_grad:
            raise E.ErrNoGrad("the loss is not differentiable with respect to the parameters")
        params = [p for _, (t, p) in trainable.items()]
        uniq = list({id(p): p for p in params}.values())
        grads = torch.autograd.grad(out, [inputs[id(p)] for p in uniq], allow_unused=True)
    fresh_dst, fresh_src, acc_dst, acc_src = [], [], [], []
    for p, g in zip(uniq, grads):
        if g is None:
            continue
        g = g.detach()
        buf = p._grad_buf
        if buf is not None and buf.shape == g.shape and buf.dtype == g.dtype and buf.device == g.device:
            # the optimizer keeps this gradient in a flat buffer: write / accumulate in place
            if p._grad is None:
                fresh_dst.append(buf)
                fresh_src.append(g)
                p._grad = buf
            else:
                acc_dst.append(p._grad)
                acc_src.append(g)
        else:
            p._grad = g if p._grad is None else p._grad + g
    if fresh_dst:
        torch._foreach_copy_(fresh_dst, fresh_src)
    if acc_dst:
        torch._foreach_add_(acc_dst, acc_src)
    for p in uniq:
        p._data.requires_grad_(False)
    loss._assign(out.detach())
    loss._fn, loss._args, loss._kw = None, (), {}
    for e, v in zip(carried, side):
        e._assign(v.detach())
        e._fn, e._args, e._kw = None, (), {}
    for e in effects:
        e()


def gradients(loss: C.Tensor, wrt) -> list:
    """Gradients of a scalar with respect to arbitrary tensors of its graph (not accumulated)."""
    wrt = list(wrt)
    memo = {}
    leaves = []
    for w in wrt:
        v = w.data().detach().clone().requires_grad_(True)
        memo[id(w)] = v
        leaves.append(v)
    with torch.enable_grad():
        (out,) = C.evaluate([loss], memo, reuse_cached=False)
        gs = torch.autograd.grad(out, leaves, allow_unused=True)
    return [C.from_torch(torch.zeros_like(l) if g is None else g) for g, l in zip(gs, leaves)]


def _wrap_fn(f):
    """Lifts a function over lazy Tensors to one over torch tensors (for torch.func)."""
    def g(*xs):
        outs = f(*[_Traced(x) for x in xs])
        if isinstance(outs, (tuple, list)):
            return tuple(_untrace(o) for o in outs)
        return _untrace(outs)
    return g


class _Traced(C.Tensor):
    """A leaf whose value is a torch.func tracer (kept out of the realized cache)."""

    def __init__(self, v):
        super().__init__(val=v, shape=v.shape, dtype=v.dtype, device=C._dev_of(v))


def _untrace(t: C.Tensor):
    if t._err is not None:
        raise t._err
    (v,) = C.evaluate([t], {}, reuse_cached=True)
    return v


def _value(x):
    """The torch value a transform starts from.  Inside another transform (a gradient under ``jvp`` or
    ``vmap``) the value is that transform's tracer and must keep its tangent or batch level, so it is
    not detached."""
    from .memory import in_transform
    return _untrace(x) if in_transform() else x.data()


def grad(f, argnums=0):
    """``grad(f)(x...)`` = gradient of the scalar ``f`` (tensor.Grad)."""
    def run(*xs):
        vals = [_value(x) for x in xs]
        out = torch.func.grad(_wrap_fn(f), argnums=argnums)(*vals)
        return tuple(C.from_torch(o) for o in out) if isinstance(out, tuple) else C.from_torch(out)
    return run


def _lift_out(o):
    """torch results (one tensor or a tuple of them) as lazy tensors."""
    return tuple(C.from_torch(v) for v in o) if isinstance(o, (tuple, list)) else C.from_torch(o)


def vjp(f, *xs):
    """``f(x...)`` (one tensor or a tuple) and the function from cotangents of the outputs to the
    gradients of the inputs (tensor.VJP)."""
    out, pull = torch.func.vjp(_wrap_fn(f), *[_value(x) for x in xs])

    def pullback(*ct):
        res = pull(tuple(_value(c) for c in ct) if isinstance(out, tuple) else _value(ct[0]))
        return tuple(C.from_torch(r) for r in res)
    return _lift_out(out), pullback


def jvp(f, xs, tangents):
    """``f(x...)`` and its derivative along ``tangents`` (tensor.JVP); ``f`` may return a tuple, as
    ``grad(g)`` of several arguments does, which makes ``jvp(grad(g), x, v)`` a Hessian-vector product."""
    out, tan = torch.func.jvp(_wrap_fn(f), tuple(_value(x) for x in xs), tuple(_value(t) for t in tangents))
    return _lift_out(out), _lift_out(tan)


def jacobian(f, x):
    return C.from_torch(torch.func.jacrev(_wrap_fn(f))(_value(x)))


def hessian(f, x):
    return C.from_torch(torch.func.hessian(_wrap_fn(f))(_value(x)))


def vmap(f, in_axes=0, out_axes=0):
    """Vectorises ``f`` over an axis (tensor.VMap with InAxes / OutAxes)."""
    def run(*xs):
        try:
            out = torch.func.vmap(_wrap_fn(f), in_dims=in_axes, out_dims=out_axes)(*[_value(x) for x in xs])
        except RuntimeError as exc:
            raise E.ErrNotBatchable(str(exc)) from exc
        return tuple(C.from_torch(o) for o in out) if isinstance(out, tuple) else C.from_torch(out)
    return run


def func(forward, backward_fn):
    """Custom differentiable operation (tensor.Func, tensor/autograd.go:785-802):
    ``forward(*torch tensors) -> torch tensor`` and ``backward_fn(inputs, output, grad) -> grads``."""
    class _F(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *xs):
            out = forward(*xs)
            ctx.save_for_backward(*xs, out)
            return out

        @staticmethod
        def backward(ctx, g):
            *xs, out = ctx.saved_tensors
            res = backward_fn(xs, out, g)
            return tuple(res) if isinstance(res, (tuple, list)) else (res,)

    def op(*ts):
        return C._node(lambda *vs: forward(*vs) if vs and vs[0].device.type == "meta" else _F.apply(*vs), ts, {}, "func")
    return op


def checkpoint(f):
    """Recomputes ``f``'s intermediates during backward instead of keeping them
    (tensor.Checkpoint, tensor/checkpoint.go:30-68)."""
    def run(*ts):
        def ev(*vs):
            if vs and vs[0].device.type == "meta":
                return _wrap_fn(f)(*vs)
            if torch.is_grad_enabled() and any(v.requires_grad for v in vs):
                import torch.utils.checkpoint as cp
                return cp.checkpoint(_wrap_fn(f), *vs, use_reentrant=False)
            return _wrap_fn(f)(*vs)
        out = C._node(ev, ts, {}, "checkpoint")
        if isinstance(out, C.Tensor) and out._err is not None:
            out._err = E.ErrCheckpoint(str(out._err)) if not isinstance(out._err, E.MimirError) else out._err
        return out
    return run
