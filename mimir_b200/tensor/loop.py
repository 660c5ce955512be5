"""Scan loops, recording / replay and tracing.

``scan(f, init, xs)`` carries state over the leading axis of ``xs``
(tensor/loop.go:27-81: ``ScanReverse``, ``ScanCheckpoint(k)``).
``record`` runs a function once and returns a ``Recording`` that replays the
same computation over new leaves without rebuilding the graph; on CUDA the
replay is a captured CUDA graph (tensor/record.go:70-184: replay returns
``ok=False`` instead of failing when shapes do not fit).
``trace`` lists the operations of a computation for exporters (tensor/trace.go:72-110).
"""
from __future__ import annotations

import torch

from . import core as C
from .autograd import _wrap_fn


def scan(f, init, xs, reverse: bool = False, checkpoint: int = 0):
    """``carry, y_t = f(carry, x_t)`` over axis 0 of ``xs``; returns (final carry, stacked ys)."""
    def run(c0, seq):
        if seq.device.type == "meta":
            c, y = _wrap_fn(f)(c0, seq[0])
            return c, y.unsqueeze(0).expand(seq.shape[0], *y.shape)
        order = range(seq.shape[0] - 1, -1, -1) if reverse else range(seq.shape[0])
        carry, ys = c0, [None] * seq.shape[0]
        step = _wrap_fn(f)
        use_cp = checkpoint > 0 and torch.is_grad_enabled()
        for n, t in enumerate(order):
            if use_cp and n % checkpoint == 0:
                import torch.utils.checkpoint as cp
                carry, y = cp.checkpoint(step, carry, seq[t], use_reentrant=False)
            else:
                carry, y = step(carry, seq[t])
            ys[t] = y
        return carry, torch.stack(ys, 0)
    return C._node(run, (init, xs), {}, "scan")


class Recording:
    """A realized computation that can be replayed over new inputs of the same shapes."""

    def __init__(self, f, inputs):
        self._f = f
        self._sig = [(tuple(x.shape), x.dtype, repr(x.device)) for x in inputs]
        self._graph = None
        self._static_in = None
        self._static_out = None
        vals = [x.data() for x in inputs]
        self._cuda = all(v.is_cuda for v in vals) and len(vals) > 0
        self.outputs = self._run(vals)

    def _run(self, vals):
        outs = self._f(*[C.from_torch(v) for v in vals])
        single = isinstance(outs, C.Tensor)
        outs = [outs] if single else list(outs)
        C.realize(*outs)
        self._single = single
        return outs

    def replay(self, *inputs):
        """Returns ``(outputs, ok)``; ``ok`` is False when the inputs do not fit the recording."""
        sig = [(tuple(x.shape), x.dtype, repr(x.device)) for x in inputs]
        if sig != self._sig:
            return None, False
        vals = [x.data() for x in inputs]
        if self._cuda:
            if self._graph is None:
                self._static_in = [v.clone() for v in vals]
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    outs = self._run(self._static_in)
                self._graph, self._static_out = g, [o.data() for o in outs]
            for s, v in zip(self._static_in, vals):
                s.copy_(v)
            self._graph.replay()
            outs = [C.from_torch(o.clone()) for o in self._static_out]
        else:
            outs = self._run(vals)
        return (outs[0] if self._single else outs), True


    def replay_into(self, dests, *inputs) -> bool:
        """Replays and writes the results over the realized tensors ``dests``; False (nothing written)
        when the inputs or the destinations do not fit (tensor.ReplayInto)."""
        outs, ok = self.replay(*inputs)
        if not ok:
            return False
        outs = [outs] if self._single else list(outs)
        dests = [dests] if isinstance(dests, C.Tensor) else list(dests)
        if len(dests) != len(outs) or any(tuple(d.shape) != tuple(o.shape) or d.dtype != o.dtype for d, o in zip(dests, outs)):
            return False
        _write_into(dests, outs)
        return True


def _write_into(dests, outs) -> None:
    """Writes ``outs`` over the memory of ``dests`` in one schedule; the ``dests`` handles then stand
    for the new values (``realize_into`` leaves a destination stale; here the caller keeps using it)."""
    outs = list(outs)
    C.realize_into(list(dests), outs)
    for d, o in zip(dests, outs):
        d._val, d._sver = o._val, o._sver


def record(f, *inputs) -> Recording:
    return Recording(f, inputs)


def record_into(dests, f, *inputs) -> Recording:
    """``record`` whose first run already lands in ``dests`` (tensor.RecordInto)."""
    r = Recording(f, inputs)
    dests = [dests] if isinstance(dests, C.Tensor) else list(dests)
    _write_into(dests, r.outputs)
    return r


class TracedGraph:
    def __init__(self, nodes, inputs, outputs):
        self.nodes, self.inputs, self.outputs = nodes, inputs, outputs

    def ops(self):
        return [n["op"] for n in self.nodes]


def trace(f, *inputs) -> TracedGraph:
    """Runs ``f`` lazily and lists its operations in topological order."""
    outs = f(*inputs)
    outs = [outs] if isinstance(outs, C.Tensor) else list(outs)
    order, seen = [], set()

    def visit(t):
        if id(t) in seen:
            return
        seen.add(id(t))
        for a in C._flatten(t._args):
            if isinstance(a, C.Tensor):
                visit(a)
        order.append(t)
    for o in outs:
        visit(o)
    ids = {id(t): i for i, t in enumerate(order)}
    nodes = [dict(id=i, op=t._opname or ("input" if any(t is x for x in inputs) else "const"), shape=t.shape,
                  dtype=t.dtype, inputs=[ids[id(a)] for a in C._flatten(t._args) if isinstance(a, C.Tensor)])
             for i, t in enumerate(order)]
    return TracedGraph(nodes, [ids.get(id(x)) for x in inputs], [ids[id(o)] for o in outs])
