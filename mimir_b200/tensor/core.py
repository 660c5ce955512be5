"""Lazy, immutable tensors with sticky errors over PyTorch.

Reference semantics (tensor/tensor.go:17-30,126-157): every operation checks
shapes and dtypes when it is *recorded* and returns a new ``Tensor`` node;
nothing runs until ``realize`` / ``data`` / ``item`` / ``backward``.  A bad
operation does not raise: it returns a tensor that carries the error, and every
tensor computed from it carries it too.  ``MIMIR_EAGER=1`` realizes each
operation as it is recorded (tensor/tensor.go:149).

Shape inference runs the recorded function on ``meta`` tensors, so the check
costs no compute; execution maps the graph onto eager PyTorch kernels (and the
native sm_100a kernels for the fused operations) in one pass with memoisation.
"""
from __future__ import annotations

import math
import os
from typing import Any, Callable, Sequence

import torch

from . import errors as E
from . import memory as _mem

float32, float16, bfloat16, int32, int64, bool_ = (torch.float32, torch.float16, torch.bfloat16,
                                                    torch.int32, torch.int64, torch.bool)
_HALF = (torch.float16, torch.bfloat16)
_FLOAT = (torch.float32, torch.float16, torch.bfloat16, torch.float64)
_EAGER = os.environ.get("MIMIR_EAGER", "") == "1"


class Device:
    """A compute device: ``Device("cpu")`` or ``Device("gpu", index)``."""

    def __init__(self, kind: str = "cpu", index: int = 0):
        kind = {"cuda": "gpu"}.get(kind, kind)
        if kind not in ("cpu", "gpu"):
            raise E.ErrDevice(f"unknown device kind {kind!r}")
        self.kind, self.index = kind, index

    @property
    def torch(self) -> torch.device:
        return torch.device("cpu") if self.kind == "cpu" else torch.device("cuda", self.index)

    def __eq__(self, o):
        return isinstance(o, Device) and (self.kind, self.index) == (o.kind, o.index)

    def __hash__(self):
        return hash((self.kind, self.index))

    def __repr__(self):
        return "cpu" if self.kind == "cpu" else f"gpu:{self.index}"


def CPU() -> Device:
    return Device("cpu")


def GPU(index: int = 0) -> Device:
    if not torch.cuda.is_available() or index >= torch.cuda.device_count():
        raise E.ErrDevice(f"gpu:{index} is not available")
    return Device("gpu", index)


def devices() -> list:
    out = [Device("cpu")]
    if torch.cuda.is_available():
        out += [Device("gpu", i) for i in range(torch.cuda.device_count())]
    return out


def auto() -> Device:
    """The device ``MIMIR_DEVICE`` names (cpu | gpu | cuda | auto), else the first GPU, else CPU
    (tensor/device.go:173-187)."""
    want = os.environ.get("MIMIR_DEVICE", "auto").lower()
    if want in ("gpu", "cuda"):
        return GPU(0)
    if want == "cpu":
        return CPU()
    return Device("gpu", 0) if torch.cuda.is_available() else Device("cpu")


_default_device = None


def default_device() -> Device:
    global _default_device
    if _default_device is None:
        _default_device = auto()
    return _default_device


def set_default_device(d: Device) -> None:
    global _default_device
    _default_device = d


def _dev_of(t: torch.Tensor) -> Device:
    return Device("cpu") if t.device.type == "cpu" else Device("gpu", t.device.index or 0)


class Tensor:
    """One node of the lazy graph (or a realized leaf)."""

    __slots__ = ("_fn", "_args", "_kw", "_val", "_err", "shape", "dtype", "device", "_stale", "_donated",
                 "_sharding", "_opname", "_effects", "_attrs", "_sver", "__weakref__")

    def __init__(self, fn=None, args=(), kw=None, val=None, err=None, shape=(), dtype=float32, device=None,
                 opname="", attrs=None):
        self._fn, self._args, self._kw = fn, args, kw or {}
        self._val, self._err = val, err
        self.shape, self.dtype = tuple(shape), dtype
        self.device = device or default_device()
        self._stale = None      # (param, version) for views of parameter storage
        self._donated = False
        self._sharding = None
        self._opname = opname
        self._effects = ()      # tensors a backward pass computes along with the gradients
        self._attrs = attrs     # op attributes the fusion planner and the layout rules read (axes, sizes)
        # version of the memory the value lives in (see tensor/memory.py); 0 while nothing was ever written over
        self._sver = _mem.version_of(val) if _mem._VERSIONS and val is not None else 0

    def _assign(self, val) -> None:
        """Gives a lazy node its value (every path that realizes a tensor ends here or in ``realize``)."""
        self._val = val
        self._sver = _mem.version_of(val) if _mem._VERSIONS else 0

    # ------------------------------------------------------------- properties
    @property
    def err(self):
        return self._err

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def numel(self) -> int:
        return math.prod(self.shape)

    def __repr__(self):
        if self._err is not None:
            return f"Tensor(error={type(self._err).__name__}: {self._err})"
        state = "realized" if self._val is not None else "lazy"
        return f"Tensor(shape={self.shape}, dtype={str(self.dtype).replace('torch.', '')}, device={self.device}, {state})"

    # --------------------------------------------------------------- realize
    def realize(self) -> "Tensor":
        realize(self)
        return self

    def data(self) -> torch.Tensor:
        """The realized value as a (detached) torch tensor."""
        realize(self)
        return self._val.detach()

    def numpy(self):
        return self.data().float().cpu().numpy() if self.dtype in _HALF else self.data().cpu().numpy()

    def item(self):
        if self.numel() != 1 and self._err is None:
            raise E.ErrShape(f"item() needs one element, tensor has shape {self.shape}")
        return self.data().reshape(()).item()

    def tolist(self):
        return self.data().cpu().tolist()

    def bytes(self) -> bytes:
        """The realized value as raw little-endian bytes in row-major order (tensor.Bytes)."""
        v = self.data().contiguous().cpu()
        return v.view(torch.uint8).numpy().tobytes() if v.numel() else b""

    def read_bytes(self, out) -> int:
        """Copies the value's bytes into a writable buffer (bytearray, memoryview, numpy); returns the count."""
        raw = self.bytes()
        memoryview(out).cast("B")[: len(raw)] = raw
        return len(raw)

    @property
    def sharding(self):
        """``(mesh, spec)`` when the tensor is one rank's block of a sharded value, else None."""
        return getattr(self, "_sharding", None)

    def donate(self) -> "Tensor":
        """Marks a realized tensor whose owner is done with it once the NEXT schedule that reads it has
        run, as a batch of inputs that a training step reads once (tensor.Donate, tensor/tensor.go:420-452;
        internal/sched/donate.go:26-60).  That schedule may read it like any other tensor; after its
        last reader the memory goes back to the pool (so later instructions of the same schedule take it
        for their results), and from the moment the schedule runs the tensor is stale: reading it, or
        computing a tensor built from it, raises ``ErrDonated``.  Read everything you need of it in
        that one schedule, or donate a copy.  A schedule refused before it starts (the memory budget)
        leaves the tensor alone.  A tensor that is not computed yet is left alone, and so is every
        tensor when operations are evaluated as they are built (``MIMIR_EAGER=1``)."""
        if self._val is not None and self._fn is None and not _EAGER:
            self._donated = True
        return self

    def to(self, device: Device) -> "Tensor":
        if self._err is not None or device == self.device:
            return self
        src = self
        # shape inference runs on meta tensors, which have no data to move
        return _node(lambda v: v if v.device.type == "meta" else v.to(device.torch), (src,), {}, "to", device=device)

    def backward(self) -> None:
        from .autograd import backward
        backward(self)

    # ------------------------------------------------------------- operators
    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __rtruediv__(self, o): return div(o, self)
    def __neg__(self): return neg(self)
    def __matmul__(self, o): return matmul(self, o)
    def __pow__(self, o): return pow_(self, o)
    def __getitem__(self, idx): return getitem(self, idx)
    def __lt__(self, o): return less(self, o)
    def __gt__(self, o): return less(o, self)
    def __le__(self, o): return logical_not(less(o, self))
    def __ge__(self, o): return logical_not(less(self, o))


def _error_tensor(err, like: Tensor | None = None) -> Tensor:
    return Tensor(err=err, shape=like.shape if like is not None else (), dtype=like.dtype if like is not None else float32,
                  device=like.device if like is not None else None)


def from_torch(t: torch.Tensor) -> Tensor:
    return Tensor(val=t, shape=t.shape, dtype=t.dtype, device=_dev_of(t))


def tensor(data, dtype=None, device: Device | None = None) -> Tensor:
    """Creates a realized leaf from Python data, a NumPy array or a torch tensor."""
    device = device or default_device()
    try:
        if torch.is_tensor(data):
            t = data.detach().to(device.torch)
            if dtype is not None:
                t = t.to(dtype)
        else:
            t = torch.as_tensor(data)
            if dtype is None:
                dtype = float32 if t.dtype.is_floating_point else (int32 if t.dtype != torch.bool else torch.bool)
            t = t.to(dtype).to(device.torch)
        return from_torch(t)
    except Exception as exc:  # noqa: BLE001 - errors are values here
        return _error_tensor(E.classify(exc))


def _first_error(args) -> Any:
    for a in args:
        if isinstance(a, Tensor):
            if a._err is not None:
                return a._err
        elif isinstance(a, (list, tuple)):
            e = _first_error(a)
            if e is not None:
                return e
    return None


def _map_args(args, f):
    out = []
    for a in args:
        if isinstance(a, Tensor):
            out.append(f(a))
        elif isinstance(a, (list, tuple)):
            out.append(type(a)(_map_args(a, f)))
        else:
            out.append(a)
    return out


def _meta_of(t: Tensor) -> torch.Tensor:
    return torch.empty(t.shape, dtype=t.dtype, device="meta")


_META_CACHE: dict = {}


def _meta_key(fn, args, kw):
    """Structural key of a shape inference: the op's code, the constants it closes over, the operand
    shapes / dtypes and the plain arguments.  None when something in there cannot be hashed (a tensor
    captured by the closure, a list argument): that inference is simply not cached."""
    try:
        cells = tuple(c.cell_contents for c in (fn.__closure__ or ()))
        cells = tuple(() if isinstance(c, (list, dict, tuple)) and not c else c for c in cells)   # empty containers are constants
        for c in cells:
            if isinstance(c, (torch.Tensor, Tensor, list, dict)):
                return None

        def sig(a):
            if isinstance(a, Tensor):
                return ("T", tuple(a.shape), a.dtype)
            if isinstance(a, (list, tuple)):
                return tuple(sig(x) for x in a)
            return a
        key = (fn.__code__, cells, getattr(fn, "__defaults__", None), tuple(sig(a) for a in args), tuple(sorted(kw.items())))
        hash(key)
        return key
    except Exception:  # noqa: BLE001 - unhashable or exotic argument
        return None


def _node(fn: Callable, args: Sequence, kw: dict, opname: str, device: Device | None = None, attrs=None, known=None) -> Tensor:
    """Records ``fn(*args, **kw)``: propagates errors, infers shape/dtype on meta tensors (the result
    of an inference is cached by structure, so a training loop pays for it once).  ``known`` =
    (shape, dtype) skips the inference for ops whose result type is plain (elementwise ops of one
    floating tensor)."""
    err = _first_error(args)
    if err is not None:
        return _error_tensor(err)
    tensors = [a for a in _flatten(args) if isinstance(a, Tensor)]
    if device is None:
        device = tensors[0].device if tensors else default_device()
        for t in tensors:
            if t.device != device:
                return _error_tensor(E.ErrDevice(f"{opname}: operands on {device} and {t.device}"))
    if known is not None:
        out = Tensor(fn=fn, args=tuple(args), kw=kw, shape=known[0], dtype=known[1], device=device, opname=opname, attrs=attrs)
        _inherit_mesh(out, tensors)
        if _EAGER and out._sharding is None:
            realize(out)
        return out
    key = _meta_key(fn, args, kw)
    meta = _META_CACHE.get(key) if key is not None else None
    if meta is None:
        try:
            meta = fn(*_map_args(args, _meta_of), **kw)
        except Exception as exc:  # noqa: BLE001
            return _error_tensor(E.classify(exc))
        if key is not None:
            if len(_META_CACHE) > 8192:
                _META_CACHE.clear()
            _META_CACHE[key] = meta
    if isinstance(meta, (tuple, list)):
        outs = tuple(Tensor(fn=_pick(fn, i), args=tuple(args), kw=kw, shape=m.shape, dtype=m.dtype, device=device,
                            opname=opname, attrs=dict(attrs or {}, part=i)) for i, m in enumerate(meta))
        for o in outs:
            _inherit_mesh(o, tensors)
        if _EAGER and outs[0]._sharding is None:
            for o in outs:
                realize(o)
        return outs
    out = Tensor(fn=fn, args=tuple(args), kw=kw, shape=meta.shape, dtype=meta.dtype, device=device, opname=opname,
                 attrs=attrs)
    _inherit_mesh(out, tensors)
    if _EAGER and out._sharding is None:
        realize(out)
    return out


ON_MESH = "on-mesh"      # second element of ``_sharding`` for a value computed from mesh leaves (layout: by analysis)


def _inherit_mesh(out: Tensor, operands) -> None:
    """A value computed from tensors that live on a device mesh lives on that mesh: realising it goes
    through the partitioner (``parallel/spmd.py``)."""
    for t in operands:
        sh = t._sharding
        if sh is not None and (sh[1] is ON_MESH or type(t).__name__ == "MeshTensor"):
            out._sharding = (sh[0], ON_MESH)
            return


def _on_mesh(t: Tensor) -> bool:
    sh = t._sharding
    return sh is not None and t._val is None and (sh[1] is ON_MESH or type(t).__name__ == "MeshTensor")


def _pick(fn, i):
    def g(*a, **k):
        return fn(*a, **k)[i]
    return g


def _flatten(args):
    for a in args:
        if isinstance(a, (list, tuple)):
            yield from _flatten(a)
        else:
            yield a


_TAKEN = 2      # value of ``Tensor._donated`` once a schedule has consumed the donation


def _check_leaf(t: Tensor):
    if t._donated == _TAKEN:
        raise E.ErrDonated("tensor was donated to an earlier schedule")
    if _mem._VERSIONS:
        _mem.check_current(t)
    if t._stale is not None:
        p, version = t._stale
        if p._version != version:
            raise E.ErrOverwritten("parameter value was overwritten by a later in-place step")


def evaluate(roots: Sequence[Tensor], memo: dict | None = None, reuse_cached: bool = True, into: dict | None = None) -> list:
    """Evaluates the graph below ``roots`` and returns torch tensors.  ``memo`` maps ``id(node)`` to a
    value that stands in for that node (how ``backward`` substitutes differentiable leaves).  The
    graph is planned into a program (fusion, slots, early release of intermediates) that is cached
    by structure: see ``tensor/plan.py``.  ``into`` maps the position of a root to a torch tensor
    whose memory the root is to be computed into (``realize_into``)."""
    from . import plan
    memo = {} if memo is None else memo
    roots = list(roots)
    prog, w = plan.schedule(roots, memo, reuse_cached)
    leaf_vals = []
    for t in w.leaves:
        if id(t) in memo:
            leaf_vals.append(memo[id(t)])
        else:
            _check_leaf(t)
            leaf_vals.append(t._val)

    def on_error(i, err):
        w.order[i]._err = err
    pool = None
    if not torch.is_grad_enabled() and not _mem.in_transform():
        dev = next((v.device for v in leaf_vals if torch.is_tensor(v)), None)
        pool = _mem.pool_for(dev) if dev is not None else None
    # donated leaves: this schedule is their last reader; their handles are stale from here on, whether
    # the schedule succeeds or not (it has started)
    donated = [i for i, t in enumerate(w.leaves) if t._donated is True and id(t) not in memo]
    for i in donated:
        t = w.leaves[i]
        t._donated = _TAKEN
        t._val = None
    outs = prog.run(leaf_vals, w.order, on_error, pool=pool, into=into, donated=donated)
    for r, v in zip(roots, outs):
        memo[id(r)] = v
    return outs


def realize(*tensors: Tensor) -> None:
    """Computes the given tensors in one pass (sched.Realize, internal/sched/sched.go:102-166)."""
    todo = [t for t in tensors if t._val is None]
    for t in tensors:
        if t._err is not None:
            raise t._err
    if any(_on_mesh(t) for t in todo):
        from ..parallel import spmd
        return spmd.realize(*tensors)
    if not todo:
        for t in tensors:
            if t._fn is None:
                _check_leaf(t)
        return
    from .memory import reserve
    reserve(todo)
    with torch.no_grad():
        vals = evaluate(todo)
    for t, v in zip(todo, vals):
        t._val = v.detach() if torch.is_tensor(v) else v
        t._fn, t._args, t._kw = None, (), {}
        if _mem._VERSIONS:
            t._sver = _mem.version_of(t._val)


# ---------------------------------------------------------------------------
# creators
# ---------------------------------------------------------------------------
def _creator(fn, shape, dtype, device, opname):
    device = device or default_device()
    shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
    if any(s < 0 for s in shape):
        return _error_tensor(E.ErrShape(f"{opname}: negative dimension in {shape}"))
    return Tensor(fn=lambda: fn(shape, dtype, device.torch), shape=shape, dtype=dtype, device=device, opname=opname)


def _volatile(t: Tensor) -> Tensor:
    """Marks a node whose executable closes over a per-call constant (a seed): the structural key of a
    schedule ignores the constant, and a cached program runs the executable of the current graph."""
    if t._fn is not None:
        t._fn._mimir_volatile = True
    return t


def zeros(shape, dtype=float32, device=None):
    return _creator(lambda s, d, dev: torch.zeros(s, dtype=d, device=dev), shape, dtype, device, "zeros")


def ones(shape, dtype=float32, device=None):
    return _creator(lambda s, d, dev: torch.ones(s, dtype=d, device=dev), shape, dtype, device, "ones")


def full(shape, value, dtype=float32, device=None):
    return _creator(lambda s, d, dev: torch.full(s, value, dtype=d, device=dev), shape, dtype, device, "full")


def arange(n, dtype=int32, device=None):
    return _creator(lambda s, d, dev: torch.arange(s[0], dtype=d, device=dev), (n,), dtype, device, "arange")


def eye(n, dtype=float32, device=None):
    return _creator(lambda s, d, dev: torch.eye(s[0], dtype=d, device=dev), (n, n), dtype, device, "eye")


def rand(shape, seed: int = 0, dtype=float32, device=None):
    """Uniform [0,1) from the Philox4x32-10 stream of ``seed`` (same values on every device)."""
    from .random import philox_uniform
    return _volatile(_creator(lambda s, d, dev: philox_uniform(s, seed, dev).to(d), shape, dtype, device, "rand"))


def randn(shape, seed: int = 0, dtype=float32, device=None):
    from .random import philox_normal
    return _volatile(_creator(lambda s, d, dev: philox_normal(s, seed, dev).to(d), shape, dtype, device, "randn"))


# ---------------------------------------------------------------------------
# elementwise
# ---------------------------------------------------------------------------
def _lift(x, like: Tensor) -> Tensor:
    """Python scalars take the dtype of the tensor operand (no promotion)."""
    if isinstance(x, Tensor):
        return x
    if isinstance(x, (int, float, bool)):
        dt = like.dtype
        if isinstance(x, float) and not dt.is_floating_point:
            dt = float32
        # constants are immutable leaves, so one device copy per (value, dtype, device) serves every
        # graph; a training loop then uploads nothing for them (and a step can be captured into a
        # CUDA graph, where host-to-device copies of pageable memory are not allowed)
        key = (type(x), x, dt, like.device)
        val = _CONSTS.get(key)
        if val is None:
            if len(_CONSTS) > 4096:
                _CONSTS.clear()
            val = _CONSTS[key] = torch.tensor(x, dtype=dt, device=like.device.torch)
        return Tensor(val=val, shape=(), dtype=dt, device=like.device)
    return tensor(x, device=like.device)


_CONSTS: dict = {}


def _binary_dtype(a: Tensor, b: Tensor, opname: str):
    """No implicit promotion except half (+) float32 -> float32 (tensor/tensor.go:48-76)."""
    if a.dtype == b.dtype:
        return a.dtype, None
    pair = {a.dtype, b.dtype}
    if float32 in pair and (pair - {float32}).issubset(set(_HALF)):
        return float32, None
    return None, E.ErrDType(f"{opname}: dtypes {a.dtype} and {b.dtype} do not mix (cast explicitly)")


_OUT_CAPABLE = {torch.add, torch.sub, torch.mul, torch.maximum, torch.minimum, torch.neg, torch.exp, torch.log, torch.sqrt,
                torch.rsqrt, torch.sin, torch.cos, torch.tanh, torch.sigmoid, torch.abs, torch.sign, torch.floor, torch.ceil,
                torch.reciprocal, torch.erf, torch.erfinv, torch.log1p, torch.expm1}


def _broadcast(p, q):
    """Broadcast of two shapes, or None when they do not fit."""
    if p == q:
        return tuple(p)
    n = max(len(p), len(q))
    p, q = (1,) * (n - len(p)) + tuple(p), (1,) * (n - len(q)) + tuple(q)
    out = []
    for x, y in zip(p, q):
        if x != y and x != 1 and y != 1:
            return None
        out.append(y if x == 1 else x)
    return tuple(out)


_BOOL_RESULT = ("less", "equal", "logical_and", "logical_or")


def _binary(opname, fn, out_bool=False):
    def op(a, b):
        like = a if isinstance(a, Tensor) else b
        a, b = _lift(a, like), _lift(b, like)
        if a._err is not None or b._err is not None:
            return _error_tensor(a._err or b._err)
        dt, err = _binary_dtype(a, b, opname)
        if err is not None:
            return _error_tensor(err)

        def run(x, y):
            if x.dtype != y.dtype:
                x, y = x.to(dt), y.to(dt)
            return fn(x, y)
        if fn in _OUT_CAPABLE:
            # the same computation into given memory: what a program uses for pooled buffers and
            # for a destination of ``realize_into``
            def run_out(x, y, out):
                if x.dtype != y.dtype:
                    x, y = x.to(dt), y.to(dt)
                fn(x, y, out=out)
            run._mimir_out = run_out
        # the result type of an elementwise op of two tensors is their broadcast shape in the common
        # dtype (comparisons: bool); shapes that do not broadcast go through the inference and come
        # back as a sticky error
        shape = _broadcast(a.shape, b.shape)
        known = None if shape is None else (shape, torch.bool if opname in _BOOL_RESULT else dt)
        return _node(run, (a, b), {}, opname, attrs={"kind": "binary"}, known=known)
    op.__name__ = opname
    return op


def _int_div(x, y):
    if not x.dtype.is_floating_point:
        if y.device.type != "meta" and bool((y == 0).any()):
            raise E.ErrDivideByZero("integer division by zero")
        return torch.div(x, y, rounding_mode="trunc")
    return x / y


add = _binary("add", torch.add)
sub = _binary("sub", torch.sub)
mul = _binary("mul", torch.mul)
div = _binary("div", _int_div)
maximum = _binary("maximum", torch.maximum)
minimum = _binary("minimum", torch.minimum)
pow_ = _binary("pow", torch.pow)
less = _binary("less", torch.lt)
equal = _binary("equal", torch.eq)
mod = _binary("mod", torch.remainder)
logical_and = _binary("logical_and", torch.logical_and)     # non-zero counts as true, like the comparisons' results
logical_or = _binary("logical_or", torch.logical_or)


def _unary(opname, fn, native_mode=None, same_type=True):
    """An elementwise op of one tensor; ``native_mode`` names the activation kernel that serves
    bf16 CUDA tensors (forward and backward) instead of the PyTorch op."""
    def op(x: Tensor, *args, **kw):
        def run(v):
            if native_mode is not None and _native_ok(v) and v.numel() % 8 == 0 and v.numel():
                from ..ops import functional as NF
                return NF.activation(v, native_mode)
            return fn(v, *args, **kw)
        if fn in _OUT_CAPABLE and native_mode is None and not args and not kw:
            def run_out(v, out):
                fn(v, out=out)
            run._mimir_out = run_out
        # an elementwise op of a floating tensor keeps its shape and dtype: no inference needed
        known = (x.shape, x.dtype) if same_type and isinstance(x, Tensor) and x._err is None and x.dtype.is_floating_point \
            and not args and not kw else None
        return _node(run, (x,), {}, opname, attrs={"kind": "unary", "plain": not args and not kw}, known=known)
    op.__name__ = opname
    return op


neg = _unary("neg", torch.neg)
exp = _unary("exp", torch.exp)
log = _unary("log", torch.log)
sqrt = _unary("sqrt", torch.sqrt)
rsqrt = _unary("rsqrt", torch.rsqrt)
sin = _unary("sin", torch.sin)
cos = _unary("cos", torch.cos)
tanh = _unary("tanh", torch.tanh)
sigmoid = _unary("sigmoid", torch.sigmoid)
relu = _unary("relu", torch.relu, "relu")
abs_ = _unary("abs", torch.abs)
sign = _unary("sign", torch.sign)
floor = _unary("floor", torch.floor)
ceil = _unary("ceil", torch.ceil)
recip = _unary("recip", torch.reciprocal)
erf = _unary("erf", torch.erf)
erfinv = _unary("erfinv", torch.erfinv)
log1p = _unary("log1p", torch.log1p)
expm1 = _unary("expm1", torch.expm1)
lgamma = _unary("lgamma", torch.lgamma)
digamma = _unary("digamma", torch.digamma)
logical_not = _unary("logical_not", torch.logical_not, same_type=False)
silu = _unary("silu", torch.nn.functional.silu, "silu")
softplus = _unary("softplus", torch.nn.functional.softplus)


def trigamma(x):
    return _node(lambda v: torch.polygamma(1, v), (x,), {}, "trigamma")


def gelu(x, approximate: str = "tanh"):
    """GELU; the tanh form is the default like the reference (tensor/elementwise.go:556-594)."""
    def run(v):
        if approximate == "tanh" and _native_ok(v) and v.numel() % 8 == 0 and v.numel():
            from ..ops import functional as NF
            return NF.activation(v, "gelu")
        return torch.nn.functional.gelu(v, approximate=approximate)
    return _node(run, (x,), {}, "gelu", attrs={"kind": "unary", "approximate": approximate})


def leaky_relu(x, slope=0.01):
    return _node(lambda v: torch.nn.functional.leaky_relu(v, slope), (x,), {}, "leaky_relu")


def clamp(x, lo=None, hi=None):
    return _node(lambda v: torch.clamp(v, lo, hi), (x,), {}, "clamp")


def where(cond, a, b):
    like = a if isinstance(a, Tensor) else b if isinstance(b, Tensor) else cond
    a, b = _lift(a, like), _lift(b, like)
    return _node(lambda c, x, y: torch.where(c.bool(), x, y.to(x.dtype)), (cond, a, b), {}, "where")


def cast(x, dtype):
    return _node(lambda v: v.to(dtype), (x,), {}, "cast", attrs={"kind": "unary"})


def _swiglu_run(g, u):
    if g.shape == u.shape and _native_ok(g, u) and g.numel() % 8 == 0 and g.numel():
        from ..ops import functional as NF
        return NF.swiglu(g, u)
    return torch.nn.functional.silu(g) * u


def swiglu(gate, up):
    """``silu(gate) * up``: one kernel (forward and backward) for bf16 CUDA tensors."""
    return _node(_swiglu_run, (gate, up), {}, "swiglu", attrs={"kind": "binary"})


# ---------------------------------------------------------------------------
# movement
# ---------------------------------------------------------------------------
def reshape(x, shape):
    return _node(lambda v: v.reshape(shape), (x,), {}, "reshape", attrs={"shape": tuple(shape)})


def permute(x, dims):
    return _node(lambda v: v.permute(dims), (x,), {}, "permute", attrs={"dims": tuple(dims)})


def transpose(x, a=-1, b=-2):
    return _node(lambda v: v.transpose(a, b), (x,), {}, "transpose", attrs={"a": a, "b": b})


def expand(x, shape):
    return _node(lambda v: v.expand(shape), (x,), {}, "expand", attrs={"shape": tuple(shape)})


def squeeze(x, dim=None):
    return _node(lambda v: v.squeeze() if dim is None else v.squeeze(dim), (x,), {}, "squeeze", attrs={"dim": dim})


def unsqueeze(x, dim):
    return _node(lambda v: v.unsqueeze(dim), (x,), {}, "unsqueeze", attrs={"dim": dim})


def flip(x, dims):
    return _node(lambda v: v.flip(dims), (x,), {}, "flip")


def pad(x, pads, value=0.0):
    """``pads`` = (before, after) per axis, first axis first."""
    flat = []
    for before, after in reversed(list(pads)):
        flat += [before, after]
    return _node(lambda v: torch.nn.functional.pad(v, flat, value=value), (x,), {}, "pad")


def shrink(x, ranges):
    """Keeps ``[lo, hi)`` of every axis (reference primitive ``Shrink``)."""
    def run(v):
        for ax, (lo, hi) in enumerate(ranges):
            if lo < 0 or hi > v.shape[ax] or lo > hi:
                raise E.ErrIndex(f"shrink: range [{lo},{hi}) outside axis {ax} of size {v.shape[ax]}")
            v = v.narrow(ax, lo, hi - lo)
        return v
    return _node(run, (x,), {}, "shrink", attrs={"ranges": tuple(tuple(r) for r in ranges)})


def getitem(x, idx):
    if isinstance(idx, Tensor):
        return gather_rows(x, idx)
    return _node(lambda v: v[idx], (x,), {}, "getitem")


def cat(xs, dim=0):
    return _node(lambda vs: torch.cat(list(vs), dim), (list(xs),), {}, "cat", attrs={"dim": dim})


def stack(xs, dim=0):
    return _node(lambda vs: torch.stack(list(vs), dim), (list(xs),), {}, "stack")


def split(x, sizes, dim=0):
    return _node(lambda v: tuple(torch.split(v, sizes, dim)), (x,), {}, "split",
                 attrs={"sizes": tuple(sizes) if isinstance(sizes, (list, tuple)) else sizes, "dim": dim})


def contiguous(x):
    return _node(lambda v: v.contiguous(), (x,), {}, "contiguous", attrs={"kind": "unary"})


def _check_index(i, n, opname):
    # a batched index (under vmap) cannot be read on the host; the torch op checks the bounds itself there
    if torch._C._functorch.is_functorch_wrapped_tensor(i):
        return
    if i.device.type != "meta" and i.numel() and (int(i.min()) < 0 or int(i.max()) >= n):
        raise E.ErrIndex(f"{opname}: index outside [0, {n})")


def gather_rows(x, index):
    """``x[index]`` along axis 0 (embedding lookup); out-of-range indices are ErrIndex."""
    def run(v, i):
        if v.dim() == 2 and _native_ok(v) and i.is_cuda and v.shape[1] % 8 == 0 and i.numel():
            # the kernel checks the range itself and reports through the device error word
            from ..ops import functional as NF
            return NF.embedding(v, i)
        _check_index(i, v.shape[0], "gather")
        return v[i.long()]
    return _node(run, (x, index), {}, "gather_rows")


def gather(x, dim, index):
    def run(v, i):
        _check_index(i, v.shape[dim], "gather")
        return torch.gather(v, dim, i.long())
    return _node(run, (x, index), {}, "gather")


def scatter_add(x, dim, index, src):
    def run(v, i, s):
        _check_index(i, v.shape[dim], "scatter_add")
        return v.scatter_add(dim, i.long(), s)
    return _node(run, (x, index, src), {}, "scatter_add")


def scatter(x, dim, index, src):
    def run(v, i, s):
        _check_index(i, v.shape[dim], "scatter")
        return v.scatter(dim, i.long(), s)
    return _node(run, (x, index, src), {}, "scatter")


def slice_scatter(x, src, dim, start, end):
    return _node(lambda v, s: torch.slice_scatter(v, s, dim, start, end), (x, src), {}, "slice_scatter")


def unfold(x, kernel, stride=1, padding=0, dilation=1):
    return _node(lambda v: torch.nn.functional.unfold(v, kernel, dilation, padding, stride), (x,), {}, "unfold")


def fold(x, output_size, kernel, stride=1, padding=0, dilation=1):
    return _node(lambda v: torch.nn.functional.fold(v, output_size, kernel, dilation, padding, stride), (x,), {}, "fold")


def one_hot(index, classes, dtype=float32):
    def run(i):
        _check_index(i, classes, "one_hot")
        return torch.nn.functional.one_hot(i.long(), classes).to(dtype)
    return _node(run, (index,), {}, "one_hot")


# ---------------------------------------------------------------------------
# reductions: half inputs accumulate in fp32 and return float32 (tensor/tensor.go:68-69)
# ---------------------------------------------------------------------------
def _reduce(opname, fn):
    def op(x, dim=None, keepdim=False):
        def run(v):
            if v.dtype in _HALF:
                v = v.float()
            return fn(v, dim, keepdim)
        return _node(run, (x,), {}, opname, attrs={"kind": "reduce", "dim": dim, "keepdim": keepdim})
    op.__name__ = opname
    return op


sum_ = _reduce("sum", lambda v, d, k: v.sum() if d is None else v.sum(d, keepdim=k))
mean = _reduce("mean", lambda v, d, k: v.mean() if d is None else v.mean(d, keepdim=k))
max_ = _reduce("max", lambda v, d, k: v.max() if d is None else v.amax(d, keepdim=k))
min_ = _reduce("min", lambda v, d, k: v.min() if d is None else v.amin(d, keepdim=k))
var = _reduce("var", lambda v, d, k: v.var(unbiased=True) if d is None else v.var(d, unbiased=True, keepdim=k))  # sample variance, like the reference
logsumexp = _reduce("logsumexp", lambda v, d, k: torch.logsumexp(v, tuple(range(v.ndim)) if d is None else d, keepdim=k))


def argmax(x, dim=-1):
    return _node(lambda v: v.argmax(dim).to(int32), (x,), {}, "argmax")


def softmax(x, dim=-1):
    return _node(lambda v: torch.softmax(v.float(), dim).to(v.dtype), (x,), {}, "softmax", attrs={"dim": dim})


def log_softmax(x, dim=-1):
    return _node(lambda v: torch.log_softmax(v.float(), dim).to(v.dtype), (x,), {}, "log_softmax", attrs={"dim": dim})


def _scan(opname, mode, fallback):
    """Running sum / maximum / log-sum-exp: the native block-per-row scan for fp32 / bf16 tensors on
    the GPU outside autograd, PyTorch otherwise."""
    def op(x, dim=-1):
        def run(v):
            if v.is_cuda and not torch.is_grad_enabled() and v.dim() >= 1:
                from ..ops import scan as native
                if native.supported(v):
                    return native.scan(v, mode, dim)
            return fallback(v, dim)
        return _node(run, (x,), {}, opname)
    op.__name__ = opname
    return op


cumsum = _scan("cumsum", "sum", lambda v, d: torch.cumsum(v, d))
cummax = _scan("cummax", "max", lambda v, d: torch.cummax(v, d).values)
logcumsumexp = _scan("logcumsumexp", "logsumexp", lambda v, d: torch.logcumsumexp(v, d))


def sort(x, dim=-1, descending=False):
    """``(values, indices)``, stable: equal values keep their order (tensor/sort.go)."""
    return _node(lambda v: tuple(torch.sort(v, dim=dim, descending=descending, stable=True)), (x,), {}, "sort")


def argsort(x, dim=-1, descending=False):
    return _node(lambda v: torch.argsort(v, dim=dim, descending=descending, stable=True).to(int32), (x,), {}, "argsort")


def topk(x, k, dim=-1, largest=True):
    """``(values, indices)`` of the ``k`` largest (or smallest) entries along ``dim``, in order."""
    return _node(lambda v: tuple(torch.topk(v, k, dim, largest=largest)), (x,), {}, "topk")


def cummax_indices(x, dim=-1):
    """Position of the running maximum along ``dim``; of equal values (or after a NaN) the latest one."""
    return _node(lambda v: torch.cummax(v, dim).indices.to(int32), (x,), {}, "cummax_indices")


def windows(x, axis, size, step=1):
    """Sliding windows of ``size`` values every ``step`` along ``axis``, as a new last axis
    (tensor.Unfold over one axis: ``[..., n, ...] -> [..., (n - size) // step + 1, ..., size]``)."""
    return _node(lambda v: v.unfold(axis, size, step), (x,), {}, "windows", attrs={"axis": axis, "size": size, "step": step})


# ---------------------------------------------------------------------------
# products
# ---------------------------------------------------------------------------
_NATIVE = os.environ.get("MIMIR_NATIVE", "1") != "0"


def _native_ok(*vals) -> bool:
    """True when every operand is a bf16 CUDA tensor and the native kernels are not switched off
    (``MIMIR_NATIVE=0`` keeps the whole layer on PyTorch library kernels: the baseline mode)."""
    return _NATIVE and all(v is not None and v.is_cuda and v.dtype == bfloat16 for v in vals)


def set_native(on: bool) -> bool:
    """Switches the native sm_100a dispatch of this layer on or off; returns the previous setting."""
    global _NATIVE
    old, _NATIVE = _NATIVE, bool(on)
    return old


def matmul(a, b):
    """``a @ b`` with batch broadcasting.  bf16 CUDA operands with a 2-D right-hand side run on the
    tcgen05 GEMM (forward, and both gradients in backward)."""
    def run(x, y):
        if x.dtype != y.dtype:
            raise E.ErrDType(f"matmul: dtypes {x.dtype} and {y.dtype} differ")
        if _native_ok(x, y) and y.dim() == 2 and x.dim() >= 2 and y.shape[1] % 8 == 0 and x.shape[-1] % 8 == 0 \
                and x.numel():
            from ..ops import functional as NF
            lead = x.shape[:-1]
            x2 = x.reshape(-1, x.shape[-1])
            out = NF.MatmulFn.apply(x2 if x2.is_contiguous() else x2.contiguous(), y if y.is_contiguous() else y.contiguous())
            return out.view(*lead, y.shape[1])
        return x @ y
    return _node(run, (a, b), {}, "matmul")


def _linear_run(act: int, has_bias: bool, has_res: bool):
    """The executable of a Linear product with an optional fused GELU-tanh (``act`` 1) or residual
    add: the native GEMM with the epilogue folded in for bf16 CUDA operands, PyTorch otherwise."""
    def run(v, wt, *rest):
        if v.dtype != wt.dtype:
            raise E.ErrDType(f"linear: input {v.dtype} and weight {wt.dtype} differ")
        b = rest[0] if has_bias else None
        r = rest[1 if has_bias else 0] if has_res else None
        extra = tuple(t for t in (b, r) if t is not None)
        if _native_ok(v, wt, *extra) and wt.dim() == 2 and wt.shape[0] % 8 == 0 and wt.shape[1] % 8 == 0 and v.numel():
            from ..ops import functional as NF
            return NF.linear(v, wt, b, r, act)
        y = torch.nn.functional.linear(v, wt, b)
        if act == 1:
            y = torch.nn.functional.gelu(y, approximate="tanh")
        return y + r if r is not None else y
    return run


def matmul_t(x, w, bias=None):
    """``x @ w^T (+ bias)``: the Linear product with the weight stored [out, in]
    (nn/layers.go:49-55).  ``w`` may be a quantized buffer."""
    from ..io.mim import QuantizedTensor
    if isinstance(w, QuantizedTensor):
        from ..ops.quant import qmatmul_t
        return _node(lambda v: qmatmul_t(v, w), (x,), {}, "qmatmul")
    args = (x, w) + ((bias,) if bias is not None else ())
    # the plain case has a plain result type; anything else (a mismatch, mixed dtypes) goes through
    # the inference, which turns it into a sticky error or a promotion
    known = None
    if isinstance(x, Tensor) and isinstance(w, Tensor) and x._err is None and w._err is None and len(w.shape) == 2 \
            and len(x.shape) >= 1 and x.shape[-1] == w.shape[1] and x.dtype == w.dtype and x.dtype.is_floating_point \
            and (bias is None or (isinstance(bias, Tensor) and bias._err is None and tuple(bias.shape) == (w.shape[0],)
                                  and bias.dtype == x.dtype)):
        known = (tuple(x.shape[:-1]) + (w.shape[0],), x.dtype)
    return _node(_linear_run(0, bias is not None, False), args, {}, "linear",
                 attrs={"bias": bias is not None, "act": 0, "residual": False}, known=known)


def attention(q, k, v, causal=False, causal_offset=None, mask=None, scale=None):
    """Fused attention over ``[B, H, T, D]`` tensors (tensor/attention.go:81-253): grouped-query
    heads when ``k``/``v`` have fewer heads, optional causal mask (query i sees keys j <= i +
    ``causal_offset``; 0 by default, so the first query sees the first key alone; a decoding step
    over a cache of Tk - Tq keys passes that many), additive or boolean mask; never materialises the score matrix on the CUDA bf16 path (forward and
    backward both run the tcgen05 kernels)."""
    args = (q, k, v) + ((mask,) if mask is not None else ())

    def run(qv, kv, vv, *m):
        B, Hq, Tq, D = qv.shape
        Hk, Tk = kv.shape[1], kv.shape[2]
        if Hq % Hk:
            raise E.ErrShape(f"attention: {Hq} query heads are not a multiple of {Hk} key heads")
        off = 0 if causal_offset is None else causal_offset
        if not m and _native_ok(qv, kv, vv) and D in (64, 128) and kv.shape == vv.shape:
            from ..ops import functional as NF
            return NF.attention(qv, kv, vv, causal=causal, offset=off, scale=scale)
        if Hk != Hq:
            kv = kv.repeat_interleave(Hq // Hk, 1)
            vv = vv.repeat_interleave(Hq // Hk, 1)
        am = None
        if causal:
            i = torch.arange(Tq, device=qv.device)[:, None]
            j = torch.arange(Tk, device=qv.device)[None]
            am = torch.zeros(Tq, Tk, device=qv.device, dtype=qv.dtype).masked_fill(j > i + off, float("-inf"))
        if m:
            mm = m[0]
            if mm.dtype == torch.bool:
                mm = torch.zeros_like(mm, dtype=qv.dtype).masked_fill(~mm, float("-inf"))
            am = mm if am is None else am + mm
        if _mem.in_transform():
            # the fused library kernel has no forward-mode derivative: under jvp / vmap / nested
            # gradients the scores are written out in ops that have every rule
            s = torch.matmul(qv, kv.transpose(-1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(D))
            return torch.matmul(torch.softmax(s if am is None else s + am, -1), vv)
        return torch.nn.functional.scaled_dot_product_attention(qv, kv, vv, attn_mask=am, scale=scale)
    return _node(run, args, {}, "attention", attrs={"causal": causal, "mask": mask is not None})


def conv2d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    """2-D convolution; stride-1 bf16 CUDA convolutions run as implicit GEMMs on the tcgen05 kernels
    (forward, input gradient and filter gradient), everything else on PyTorch."""
    args = (x, w) + ((bias,) if bias is not None else ())

    def run(v, wt, *b):
        if _native_ok(v, wt, *b):
            from ..ops import functional as NF
            if NF.conv2d_supported(v, wt, stride, padding, dilation, groups):
                return NF.conv2d(v, wt, b[0] if b else None, padding, dilation)
        return torch.nn.functional.conv2d(v, wt, b[0] if b else None, stride, padding, dilation, groups)
    return _node(run, args, {}, "conv2d")


def conv1d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    args = (x, w) + ((bias,) if bias is not None else ())
    return _node(lambda v, wt, *b: torch.nn.functional.conv1d(v, wt, b[0] if b else None, stride, padding, dilation, groups),
                 args, {}, "conv1d")


def conv3d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    args = (x, w) + ((bias,) if bias is not None else ())
    return _node(lambda v, wt, *b: torch.nn.functional.conv3d(v, wt, b[0] if b else None, stride, padding, dilation, groups),
                 args, {}, "conv3d")


def conv_transpose2d(x, w, bias=None, stride=1, padding=0, output_padding=0):
    args = (x, w) + ((bias,) if bias is not None else ())
    return _node(lambda v, wt, *b: torch.nn.functional.conv_transpose2d(v, wt, b[0] if b else None, stride, padding, output_padding),
                 args, {}, "conv_transpose2d")


def conv_transpose1d(x, w, bias=None, stride=1, padding=0, output_padding=0):
    args = (x, w) + ((bias,) if bias is not None else ())
    return _node(lambda v, wt, *b: torch.nn.functional.conv_transpose1d(v, wt, b[0] if b else None, stride, padding, output_padding),
                 args, {}, "conv_transpose1d")


def max_pool2d(x, kernel, stride=None, padding=0):
    def run(v):
        if _native_ok(v):
            from ..ops import functional as NF
            if NF.max_pool2d_supported(v, kernel, stride, padding):
                return NF.max_pool2d(v, kernel, stride)
        return torch.nn.functional.max_pool2d(v, kernel, stride, padding)
    return _node(run, (x,), {}, "max_pool2d")


def avg_pool2d(x, kernel, stride=None, padding=0):
    return _node(lambda v: torch.nn.functional.avg_pool2d(v, kernel, stride, padding), (x,), {}, "avg_pool2d")


def upsample_nearest(x, scale):
    return _node(lambda v: torch.nn.functional.interpolate(v, scale_factor=scale, mode="nearest"), (x,), {}, "upsample")


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    """Normalises over the last axis; ``weight`` / ``bias`` of that length are optional."""
    n = x.shape[-1] if x.shape else 1
    extra = tuple(t for t in (weight, bias) if t is not None)
    hw, hb = weight is not None, bias is not None

    def run(v, *wb):
        w = wb[0] if hw else None
        b = wb[1 if hw else 0] if hb else None
        if hw and hb and _native_ok(v, w, b) and n % 8 == 0 and n <= 8192 and v.numel():
            from ..ops import functional as NF
            return NF.layer_norm(v, w, b, eps)
        return torch.nn.functional.layer_norm(v, (n,), w, b, eps)
    return _node(run, (x, *extra), {}, "layer_norm", attrs={"kind": "rowwise"})


def rms_norm(x, weight=None, eps: float = 1e-6):
    """Root-mean-square normalisation over the last axis in fp32, rounded to the input dtype, then
    scaled by ``weight``."""
    def run(v, *w):
        if w and _native_ok(v, w[0]) and v.shape[-1] % 8 == 0 and v.shape[-1] <= 8192 and v.numel():
            from ..ops import functional as NF
            return NF.rms_norm(v, w[0], eps)
        y = (v.float() * torch.rsqrt(v.float().pow(2).mean(-1, keepdim=True) + eps)).to(v.dtype)
        return y * w[0] if w else y
    return _node(run, (x,) + ((weight,) if weight is not None else ()), {}, "rms_norm", attrs={"kind": "rowwise"})


def with_effects(x, *effects):
    """``x`` with the same values and gradients, carrying ``effects``: tensors that ``backward``
    computes in the same schedule as the gradients whenever it runs on a result computed from the
    returned tensor (tensor/autograd.go:753-777).  Layers use it for state a training step updates on
    the side (the running statistics of batch normalisation), so the update costs no extra pass.
    Gradients and the transformations ignore effects."""
    for e in effects:
        if isinstance(e, Tensor) and e._err is not None:
            return _error_tensor(e._err)
    if not effects:
        return x
    out = _node(lambda v: v, (x,), {}, "with_effects")
    if out._err is None:
        out._effects = tuple(effects)
    return out


def detach(x):
    """The same values with no gradient flowing back (tensor.Detach)."""
    return _node(lambda v: v.detach(), (x,), {}, "detach", attrs={"kind": "unary"})


def from_bytes(data, shape, dtype=torch.float32, device: Device | None = None) -> Tensor:
    """A tensor over raw little-endian bytes (bytes, bytearray, memoryview, mmap) without copying when
    the buffer is writable or the target is another device (tensor.FromBytes, tensor/bytes.go)."""
    shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
    need = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
    mv = memoryview(data).cast("B")
    if len(mv) < need:
        return _error_tensor(E.ErrShape(f"from_bytes: {len(mv)} bytes for shape {shape} of {dtype} ({need} needed)"))
    import numpy as np
    arr = np.frombuffer(mv, dtype=np.uint8, count=need)
    t = torch.from_numpy(arr if arr.flags.writeable else arr.copy()).view(dtype).view(shape)
    return from_torch(t if device is None else t.to(device.torch))


def from_bytes_func(fill, shape, dtype=torch.float32, device: Device | None = None) -> Tensor:
    """Like ``from_bytes`` but ``fill(buffer)`` writes the bytes into storage this call owns (one copy
    fewer when the source is a stream)."""
    shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
    t = torch.empty(shape, dtype=dtype)
    fill(memoryview(t.view(torch.uint8).numpy()).cast("B"))
    return from_torch(t if device is None else t.to(device.torch))


def realize_into(dsts, srcs):
    """Computes every tensor of ``srcs`` in ONE schedule and writes ``srcs[i]`` over the memory of the
    realized tensor ``dsts[i]`` (same shape, dtype and device; ``None`` = new memory) where it can,
    as an optimizer writes a parameter's new value over the old one (tensor.RealizeInto,
    tensor/tensor.go:356-378; internal/sched/into.go:24-66).  Both may be single tensors.

    Afterwards ``srcs[i]`` is realized IN the memory of ``dsts[i]``, and ``dsts[i]`` is stale, and so is
    every tensor realized earlier that shares its memory (a view): reading one, or computing a tensor
    built from one, raises ``ErrOverwritten``.  The value is computed straight into the destination
    when the instruction that produces it can write into given memory (elementwise ops) and nothing
    in the schedule reads the old values after it; otherwise it is computed into pooled memory and
    copied over when the schedule has finished reading.  On error nothing is written."""
    single = isinstance(srcs, Tensor)
    dsts = [dsts] if single else list(dsts)
    srcs = [srcs] if single else list(srcs)
    if len(dsts) != len(srcs):
        raise E.ErrShape(f"realize_into: {len(dsts)} destinations for {len(srcs)} tensors")
    seen = set()
    for d, s in zip(dsts, srcs):
        if s._err is not None:
            raise s._err
        if d is None:
            continue
        if d._val is None:
            raise E.ErrNilTensor("realize_into: the destination is not realized")
        _check_leaf(d)
        if tuple(d.shape) != tuple(s.shape) or d.dtype != s.dtype or d.device != s.device:
            raise E.ErrShape(f"realize_into: {tuple(s.shape)} {s.dtype} on {s.device} does not fit "
                             f"{tuple(d.shape)} {d.dtype} on {d.device}")
        if not d._val.is_contiguous():
            raise E.ErrUnsupported("realize_into: the destination is a strided view")
        a = _mem._address(d._val)
        if a in seen:
            raise E.ErrOverwritten("realize_into: two destinations share memory")
        seen.add(a)
    todo = [(i, s) for i, s in enumerate(srcs) if s._val is None]
    if any(_on_mesh(s) for _, s in todo):
        raise E.ErrUnsupported("realize_into: tensors on a device mesh are written by the sharded step")
    if todo:
        from .memory import reserve
        reserve([s for _, s in todo])
        into = {k: dsts[i]._val for k, (i, _) in enumerate(todo) if dsts[i] is not None}
        with torch.no_grad():
            vals = evaluate([s for _, s in todo], into=into)
        for (i, s), v in zip(todo, vals):
            s._val = v.detach() if torch.is_tensor(v) else v
            s._fn, s._args, s._kw = None, (), {}
            if _mem._VERSIONS:
                # fresh memory may sit at an address that an older, overwritten storage had
                s._sver = _mem.version_of(s._val)
    for d, s in zip(dsts, srcs):
        if d is None:
            continue
        if s._val.data_ptr() != d._val.data_ptr() or _mem._address(s._val) != _mem._address(d._val):
            d._val.copy_(s._val)          # computed elsewhere (or realized before): copy, then live there
            s._val = d._val
        s._sver = _mem.overwrite(d._val)   # d (and older views of its memory) are stale from here on
    return srcs[0] if single else srcs


def _bind_methods():
    """Method forms of the functional ops (``x.sum(0)`` = ``sum_(x, 0)``), bound once; a name the
    class already defines is left alone."""
    g = globals()
    names = {"sum": "sum_", "max": "max_", "min": "min_", "abs": "abs_", "pow": "pow_"}
    for n in ("mean var logsumexp argmax softmax log_softmax cumsum exp log sqrt rsqrt sin cos tanh sigmoid relu "
              "neg sign floor ceil erf silu softplus gelu clamp cast reshape permute transpose expand squeeze "
              "unsqueeze flip pad cat contiguous gather scatter_add sort argsort topk matmul maximum minimum "
              "where one_hot with_effects detach").split():
        names[n] = n
    for meth, fn in names.items():
        if fn in g and not hasattr(Tensor, meth):
            setattr(Tensor, meth, g[fn])


# ------------------------------------------------------------------ op tracing
# While a trace is active every OUTERMOST call of a public op of this module is reported as
# (name, args, kwargs, result): what the graph exporter translates.  Ops that an op calls inside
# are not reported.  Inactive, the wrapper costs one global read per call.
_TRACE = None
_TRACE_DEPTH = 0
_NOT_OPS = {"CPU", "GPU", "devices", "auto", "default_device", "set_default_device", "from_torch", "tensor",
            "evaluate", "realize", "from_bytes", "from_bytes_func", "realize_into", "trace_ops", "set_native"}


def _traced(name, f):
    import functools

    @functools.wraps(f)
    def g(*a, **k):
        global _TRACE_DEPTH
        tr = _TRACE
        if tr is None:
            return f(*a, **k)
        _TRACE_DEPTH += 1
        try:
            out = f(*a, **k)
        finally:
            _TRACE_DEPTH -= 1
        if _TRACE_DEPTH == 0:
            tr(name, a, k, out)
        return out
    g._untraced = f
    return g


def _install_trace_hooks():
    import types
    g = globals()
    for name, f in list(g.items()):
        if name.startswith("_") or name in _NOT_OPS or not isinstance(f, types.FunctionType):
            continue
        g[name] = _traced(name, f)


class trace_ops:
    """Context manager: ``with trace_ops(callback):`` reports every outermost op call to ``callback``."""

    def __init__(self, callback):
        self.cb = callback

    def __enter__(self):
        global _TRACE, _TRACE_DEPTH
        if _TRACE is not None:
            raise RuntimeError("an op trace is already active")
        _TRACE, _TRACE_DEPTH = self.cb, 0
        return self

    def __exit__(self, *a):
        global _TRACE
        _TRACE = None


_install_trace_hooks()
_bind_methods()
