"""Memory budget: refuse a schedule before it runs when its estimate exceeds the
budget (reference: internal/sched/budget.go:26-170, tensor/device.go:213-226).

The estimate walks the unrealized graph and sums the byte sizes of every value
the pass will materialise (an upper bound: the executor frees intermediates as
their last reader finishes).  ``ErrMemoryBudget`` is raised before any kernel of
the schedule is launched, so a refused step leaves no partial state.
"""
from __future__ import annotations

import torch

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
