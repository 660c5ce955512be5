"""Python side of the C ABI over framework objects (``csrc/capi/mimir_capi.c``).

The reference is driven from Go through plain C entry points loaded with ``purego`` (no cgo:
backend/cuda/driver_linux.go:105-150; public entry points mimir.go:36-49).  The native library
of this package exports its kernels the same way; this module is the other half: tensors,
parameters, modules, optimizers and meshes as opaque 64-bit handles, every operation of the
lazy tensor layer reachable by name, errors as values.  The C shim embeds the interpreter (or
attaches to a running one), passes handles, integers, doubles, strings and raw pointers, and never
sees a Python object.

Conventions: a handle is a positive integer; 0 means failure, and ``last_error()`` then says why.
A *tensor* handle may also carry a sticky error (a bad op does not fail the call: it returns a
tensor whose error ``tensor_error`` reports, and everything computed from it carries it too), as in
the reference's tensor API (tensor/tensor.go:126-157).
"""
from __future__ import annotations

import ctypes
import json
import threading

import torch

_lock = threading.Lock()
_objects: dict = {}
_next = [1]
_last_error = [""]


def _put(obj) -> int:
    with _lock:
        h = _next[0]
        _next[0] += 1
        _objects[h] = obj
    return h


def _get(h: int):
    try:
        return _objects[h]
    except KeyError:
        raise KeyError(f"handle {h} is not live") from None


def release(h: int) -> int:
    with _lock:
        return 0 if _objects.pop(h, None) is not None else -1


def live_handles() -> int:
    return len(_objects)


def last_error() -> str:
    return _last_error[0]


def _fail(exc) -> int:
    _last_error[0] = f"{type(exc).__name__}: {exc}"
    return 0


def _device(name: str):
    from . import tensor as T
    if not name or name == "default":
        return T.default_device()
    if name == "cpu":
        return T.CPU()
    if name.startswith("gpu"):
        return T.GPU(int(name[4:] or 0) if ":" in name else 0)
    raise ValueError(f"unknown device {name!r}")


def tensor_from_memory(ptr: int, dims, dtype: str, device: str) -> int:
    """A tensor copied from ``numel`` elements at address ``ptr`` (float32 or int64)."""
    try:
        from . import tensor as T
        dims = [int(d) for d in dims]
        n = 1
        for d in dims:
            n *= d
        ctype, tdtype = {"f32": (ctypes.c_float, torch.float32), "i64": (ctypes.c_int64, torch.int64)}[dtype]
        buf = (ctype * max(n, 1)).from_address(ptr) if n else (ctype * 1)()
        t = torch.frombuffer(buf, dtype=tdtype, count=n).clone().reshape(dims)
        return _put(T.tensor(t, device=_device(device)))
    except Exception as exc:  # noqa: BLE001 - errors cross the ABI as values
        return _fail(exc)


def _resolve(name: str):
    from . import nn, optim
    from . import tensor as T
    from .nn import loss as L
    space, _, leaf = name.partition(".")
    table = {"T": T, "nn": nn, "loss": L, "optim": optim}
    if space not in table or not leaf or leaf.startswith("_"):
        raise KeyError(f"no entry point {name!r}")
    return getattr(table[space], leaf)


def call(name: str, handles, kwargs_json: str) -> int:
    """``name``: ``T.<op>`` (any public tensor op), ``nn.<Layer>`` (constructor), ``loss.<fn>``,
    ``forward`` (module, inputs...), ``parameters`` (module -> handle of the list), ``value`` / ``grad``
    (parameter -> tensor), ``item`` (list handle, index given as kwargs {"index": i})."""
    try:
        args = [_get(h) for h in handles]
        kw = json.loads(kwargs_json) if kwargs_json else {}
        if name == "forward":
            out = args[0](*args[1:], **kw)
        elif name == "parameters":
            out = list(args[0].parameters())
        elif name == "value":
            out = args[0].value()
        elif name == "grad":
            out = args[0].grad()
            if out is None:
                raise ValueError("the parameter has no gradient")
        elif name == "item":
            out = args[0][int(kw["index"])]
        elif name == "len":
            return len(args[0])
        else:
            if "dtype" in kw:
                kw["dtype"] = getattr(torch, kw["dtype"])
            out = _resolve(name)(*args, **kw)
        if isinstance(out, tuple):
            out = list(out)
        return _put(out)
    except Exception as exc:  # noqa: BLE001
        return _fail(exc)


def tensor_dims(h: int):
    try:
        return [int(d) for d in _get(h).shape]
    except Exception as exc:  # noqa: BLE001
        _fail(exc)
        return None


def tensor_error(h: int) -> str:
    """"" when the tensor carries no error, else its message (never raises)."""
    try:
        e = _get(h).err
        return "" if e is None else f"{type(e).__name__}: {e}"
    except Exception as exc:  # noqa: BLE001
        return f"{type(exc).__name__}: {exc}"


def tensor_read_f32(h: int, ptr: int, cap: int) -> int:
    """Realizes the tensor and copies it as float32 to ``ptr`` (room for ``cap`` elements); returns
    the element count, or -1 with the error recorded."""
    try:
        v = _get(h).data().detach().to("cpu", torch.float32).contiguous().reshape(-1)
        if v.numel() > cap:
            raise ValueError(f"{v.numel()} elements do not fit a buffer of {cap}")
        if v.numel():
            ctypes.memmove(ptr, v.data_ptr(), v.numel() * 4)
        return int(v.numel())
    except Exception as exc:  # noqa: BLE001
        _fail(exc)
        return -1


def backward(h: int) -> int:
    try:
        _get(h).backward()
        return 0
    except Exception as exc:  # noqa: BLE001
        _fail(exc)
        return -1


def optimizer(kind: str, module_h: int, lr: float, kwargs_json: str) -> int:
    try:
        from . import optim
        kw = json.loads(kwargs_json) if kwargs_json else {}
        return _put(getattr(optim, kind)(_get(module_h).parameters(), lr=lr, **kw))
    except Exception as exc:  # noqa: BLE001
        return _fail(exc)


def optimizer_step(h: int, zero: int) -> int:
    try:
        o = _get(h)
        o.step()
        if zero:
            o.zero_grad()
        return 0
    except Exception as exc:  # noqa: BLE001
        _fail(exc)
        return -1


def mesh(shape, axes) -> int:
    try:
        from .parallel.mesh import Mesh
        return _put(Mesh(tuple(int(s) for s in shape), tuple(axes)))
    except Exception as exc:  # noqa: BLE001
        return _fail(exc)
