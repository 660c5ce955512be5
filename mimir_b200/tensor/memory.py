"""Memory of the lazy layer: budget, storage versions, the buffer pool.

**Budget**: refuse a schedule before it runs when its estimate exceeds the
budget (reference: internal/sched/budget.go:26-170, tensor/device.go:213-226).

The estimate walks the unrealized graph and sums the byte sizes of every value
the pass will materialise (an upper bound: the executor frees intermediates as
their last reader finishes).  ``ErrMemoryBudget`` is raised before any kernel of
the schedule is launched, so a refused step leaves no partial state.

**Storage versions** (internal/graph/graph.go:86-115, internal/sched/into.go:24-38): memory that
``realize_into`` writes over gets a new version; every realized tensor remembers the version its
memory had when it was realized, so the destination and any view of its memory realized earlier are
stale afterwards (``ErrOverwritten`` when read or when a tensor built from them is computed), while
the source of the write, which now lives in that memory, is current.  Versions are kept per storage
address and only for storages that were ever written over: a program that never calls
``realize_into`` pays one empty-dict test per leaf.

**Pool** (internal/sched/memory.go:144-190, :252-304): free lists of buffers keyed by (device, dtype, element
count); a buffer that no schedule has taken for 16 schedules is released.  A program running without autograd takes the outputs of its elementwise instructions from
the pool and gives each buffer back when the last value that lives in it (the output itself or a
view some later instruction made of it) has been dropped, most recently freed first, so a replayed
schedule runs over the same buffers every time.  A buffer that a result takes away leaves the pool.
On CUDA devices PyTorch's caching allocator already is such a pool (and a captured step owns a
private one), so this pool serves CPU tensors unless ``MIMIR_POOL=all``; ``MIMIR_POOL=0`` turns it
off.
"""
from __future__ import annotations

import torch

import os

from . import errors as E

_budget = {}  # device repr -> bytes


def set_memory_budget(device, nbytes: int | None) -> None:
    if nbytes is None:
        _budget.pop(repr(device), None)
    else:
        _budget[repr(device)] = int(nbytes)


def memory_budget(device):
    return _budget.get(repr(device))


def estimate(roots) -> dict:
    """Bytes per device that realising ``roots`` will materialise."""
    from .core import Tensor, _flatten
    seen, total = set(), {}
    stack = list(roots)
    while stack:
        t = stack.pop()
        if id(t) in seen or t._val is not None or t._fn is None:
            continue
        seen.add(id(t))
        size = t.numel() * torch.empty((), dtype=t.dtype).element_size()
        total[repr(t.device)] = total.get(repr(t.device), 0) + size
        stack.extend(a for a in _flatten(t._args) if isinstance(a, Tensor))
    return total


def reserve(roots) -> None:
    if not _budget:
        return
    for dev, need in estimate(roots).items():
        limit = _budget.get(dev)
        if limit is not None and need > limit:
            raise E.ErrMemoryBudget(f"schedule needs about {need} bytes on {dev}, budget is {limit}")


def memory_of(device) -> int:
    """Bytes currently held on ``device`` by the caching allocator."""
    if device.kind == "gpu":
        return torch.cuda.memory_allocated(device.index)
    return 0


# ---------------------------------------------------------------------------
# storage versions
# ---------------------------------------------------------------------------
_VERSIONS: dict = {}    # storage address -> version, only for storages that were written over


def _address(v) -> int:
    try:
        return v.untyped_storage().data_ptr()
    except (NotImplementedError, RuntimeError):     # a transform's wrapper tensor has no storage of its own
        return 0


def version_of(v) -> int:
    """Current version of the memory a torch tensor lives in (0 until it is first written over)."""
    if not _VERSIONS or not torch.is_tensor(v) or v.device.type == "meta":
        return 0
    return _VERSIONS.get(_address(v), 0)


def overwrite(v) -> int:
    """Marks the memory of ``v`` as written over: everything realized there before is stale.
    Returns the new version."""
    a = _address(v)
    _VERSIONS[a] = n = _VERSIONS.get(a, 0) + 1
    return n


def in_transform() -> bool:
    """True inside vmap / jvp / grad transforms, whose wrapper tensors cannot be written into."""
    try:
        return torch._C._functorch.peek_interpreter_stack() is not None
    except AttributeError:
        return False


def check_current(t) -> None:
    """Raises ``ErrOverwritten`` when the memory of the realized tensor ``t`` was written over after
    ``t`` was realized."""
    if _VERSIONS and t._val is not None and torch.is_tensor(t._val) and _VERSIONS.get(_address(t._val), 0) != t._sver:
        raise E.ErrOverwritten("tensor's memory was written over by a later realize_into")


# ---------------------------------------------------------------------------
# pool
# ---------------------------------------------------------------------------
class Pool:
    """Free lists of buffers keyed by (device, dtype, element count)."""

    AGE_OUT = 16           # a buffer no schedule has asked for in this many schedules goes back to the allocator

    def __init__(self, limit_bytes: int = 1 << 30):
        self.free: dict = {}   # key -> [(buffer, schedule it was freed in), ...], most recently freed last
        self.clock = 0
        self.limit = limit_bytes
        self.held = 0          # bytes on the free lists
        self.obtained = 0      # bytes asked from the allocator
        self.reused = 0        # takes served from a free list
        self.taken = 0

    def take(self, shape, dtype, device) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= int(d)
        key = (device, dtype, n)
        lst = self.free.get(key)
        self.taken += 1
        if lst:
            buf, _ = lst.pop()
            self.held -= buf.numel() * buf.element_size()
            self.reused += 1
            return buf.view(shape)
        buf = torch.empty(n, dtype=dtype, device=device)
        self.obtained += n * buf.element_size()
        return buf.view(shape)

    def give(self, buf: torch.Tensor) -> None:
        nbytes = buf.numel() * buf.element_size()
        if self.held + nbytes > self.limit:
            return             # over the limit: the allocator gets it back
        self.held += nbytes
        self.free.setdefault((buf.device, buf.dtype, buf.numel()), []).append((buf.reshape(-1), self.clock))

    def tick(self) -> None:
        """Called once per schedule: buffers freed more than ``AGE_OUT`` schedules ago are released."""
        self.clock += 1
        if self.clock % self.AGE_OUT or not self.free:
            return
        old = self.clock - self.AGE_OUT
        for key in list(self.free):
            lst = self.free[key]
            keep = [(b, t) for b, t in lst if t >= old]
            if len(keep) != len(lst):
                self.held -= sum(b.numel() * b.element_size() for b, t in lst if t < old)
                if keep:
                    self.free[key] = keep
                else:
                    del self.free[key]

    def trim(self) -> None:
        self.free.clear()
        self.held = 0

    def stats(self) -> dict:
        return {"held_bytes": self.held, "obtained_bytes": self.obtained, "takes": self.taken, "reused": self.reused,
                "buffers": sum(len(v) for v in self.free.values())}


_POOL = Pool()
_POOL_MODE = os.environ.get("MIMIR_POOL", "cpu").lower()


def pool() -> Pool:
    return _POOL


def set_pool(mode: str) -> None:
    """``"cpu"`` (default), ``"all"`` or ``"0"``."""
    global _POOL_MODE
    _POOL_MODE = str(mode).lower()
    if _POOL_MODE in ("0", "off", "false"):
        _POOL.trim()


def pool_for(device: torch.device):
    """The pool that serves ``device`` in the current mode, or None."""
    if _POOL_MODE in ("0", "off", "false"):
        return None
    if device.type == "cpu" or _POOL_MODE == "all":
        return _POOL
    return None
