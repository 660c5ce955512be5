"""Schedules: structural keys, the fusion planner, compiled programs and their cache.

A realisation (``realize`` / ``backward``) does not interpret the lazy graph node by node.
It walks the graph once, numbering nodes and leaves and emitting a *structural key*: the
operations (code identity and the constants they close over), operand wiring, shapes,
dtypes and devices, but no tensor *values*.  Graphs built by the same model code on a new
batch have the same key, so the second step of a training loop finds a compiled
``Program`` in the cache and runs its instruction list; only a new structure pays for
planning (reference: internal/sched/key.go:181-231 structural key, cache.go:22-104 program
cache of at most 64 entries, program.go:115-355 slot-based programs).

Planning is where fusion happens (internal/sched/fuse.go:200-362).  Patterns folded here:

* ``gelu(linear(x, w, b))``           -> one GEMM with the GELU-tanh epilogue,
* ``linear(x, w, b) + r`` / ``r + linear``  -> one GEMM with the residual-add epilogue,
* ``silu(g) * u``                     -> one SwiGLU kernel,

each only when the inner value has no other reader, exactly the reference's "a node joins
its consumer when all its users share one root" rule.  The fused executables fall back to
the composed PyTorch ops when the operands are not bf16 CUDA tensors, so planning is
device-independent and the key does not need the device capabilities.

A program frees every intermediate after its last reader (the reference's pooled-buffer
"give" events) unless autograd keeps it alive.
"""
from __future__ import annotations

import collections
import os

import torch

from . import errors as E

_MAX_PROGRAMS = 64
_CACHE: "collections.OrderedDict[tuple, Program]" = collections.OrderedDict()
_STATS = {"compiled": 0, "hits": 0, "uncacheable": 0, "fused": 0, "into_direct": 0}


def compiled() -> int:
    """How many programs have been planned so far (tests use it to see cache hits: sched.Compiled)."""
    return _STATS["compiled"]


def stats() -> dict:
    return dict(_STATS, cached=len(_CACHE))


def clear_cache() -> None:
    _CACHE.clear()


class _Ref:
    """Operand of an instruction: the value in ``slot`` of the running program."""
    __slots__ = ("slot",)

    def __init__(self, slot):
        self.slot = slot


class Program:
    """A planned schedule: ``instrs`` = (fn, operand spec, kwargs, output slot, node index);
    ``nleaves`` leaf slots come first, ``roots`` are the slots to return, ``last_use[slot]`` is
    the instruction after which the slot is dropped."""

    __slots__ = ("instrs", "nleaves", "nslots", "roots", "drop_after", "fused", "out_meta", "last_use", "writer")

    def __init__(self, instrs, nleaves, nslots, roots, fused, out_meta=None):
        self.instrs, self.nleaves, self.nslots, self.roots, self.fused = instrs, nleaves, nslots, roots, fused
        self.out_meta = out_meta or [None] * len(instrs)     # (shape, dtype) of each instruction's result
        keep = set(roots)
        last = {}
        for i, (_, spec, _, _, _) in enumerate(instrs):
            for s in _spec_slots(spec):
                last[s] = i
        self.last_use = last
        self.writer = {out: i for i, (_, _, _, out, _) in enumerate(instrs)}
        self.drop_after = [[] for _ in instrs]
        for s, i in last.items():
            if s not in keep and s >= nleaves:
                self.drop_after[i].append(s)

    def run(self, leaf_vals, order=None, on_error=None, pool=None, into=None, donated=()):
        """Runs the instructions over ``leaf_vals``.  ``order`` is the node list of the graph being
        run: instructions whose executable is volatile take it from there.  ``pool`` (only without
        autograd) serves the outputs of instructions that can write into given memory; ``into`` maps
        a position in ``roots`` to the torch tensor that root is to be written into."""
        slots = list(leaf_vals) + [None] * (self.nslots - self.nleaves)
        dest = self._destinations(leaf_vals, into) if into else {}
        # a donated leaf is dropped after its last reader; its memory goes to the pool when the tensor
        # owns all of it (not a view, not a mapped file) and no result of this schedule lives in it
        drop_leaf = {}
        for s in donated:
            if s not in self.roots:
                drop_leaf.setdefault(self.last_use.get(s, -1), []).append(s)
        if pool is not None:
            pool.tick()
        owner = {} if pool is not None else None     # storage address of a pooled buffer -> [buffer, live slots]
        lives = {} if pool is not None else None     # slot -> addresses of the pooled buffers its value lives in
        for i, (fn, spec, kw, out, node_idx) in enumerate(self.instrs):
            if order is not None and getattr(fn, "_mimir_volatile", False):
                fn = order[node_idx]._fn
            try:
                writes = getattr(fn, "_mimir_out", None) if (pool is not None or i in dest) else None
                buf = None
                if writes is not None and not kw and self.out_meta[i] is not None:
                    if i in dest and self._aliased_later(slots, dest[i], i):
                        del dest[i]       # a view of the destination's memory is still to be read: copy at the end
                    if i in dest:
                        buf = dest[i]
                        _STATS["into_direct"] += 1
                    elif pool is not None:
                        shape, dtype = self.out_meta[i]
                        buf = pool.take(shape, dtype, _device_of(slots, spec))
                        owner[buf.untyped_storage().data_ptr()] = [buf, 0]
                if buf is not None:
                    writes(*_fill(spec, slots), out=buf)
                    slots[out] = buf
                else:
                    slots[out] = fn(*_fill(spec, slots), **kw)
            except E.MimirError as err:
                if on_error is not None:
                    on_error(node_idx, err)
                raise
            except Exception as exc:  # noqa: BLE001 - errors are values at the API surface
                if type(exc).__module__.startswith("torch.utils.checkpoint"):
                    raise  # control flow of activation recomputation, not a failure
                err = E.classify(exc)
                if on_error is not None:
                    on_error(node_idx, err)
                raise err from exc
            if owner:
                # a value that lives in a pooled buffer (the output itself or a view an instruction
                # made of one) keeps that buffer out of the pool until its slot is dropped
                addrs = [a for a in _addresses(slots[out]) if a in owner]
                if addrs:
                    lives[out] = addrs
                    for a in addrs:
                        owner[a][1] += 1
            for s in drop_leaf.get(i, ()):
                v, slots[s] = slots[s], None
                if pool is not None and torch.is_tensor(v) and _sole_owner(v) and not self._lives_on(slots, v):
                    pool.give(v)
                del v
            for s in self.drop_after[i]:
                slots[s] = None
                if lives and s in lives:
                    for a in lives.pop(s):
                        rec = owner[a]
                        rec[1] -= 1
                        if rec[1] == 0:
                            pool.give(rec[0])
                            del owner[a]
        # buffers that a result lives in leave the pool; the rest of what is still out goes back
        if owner:
            kept = set()
            for r in self.roots:
                kept.update(lives.get(r, ()))
            for a, rec in owner.items():
                if a not in kept:
                    pool.give(rec[0])
        return [slots[r] for r in self.roots]

    def _lives_on(self, slots, v) -> bool:
        """True when a value still held by the running program lives in the memory of ``v`` (a view some
        instruction made of it)."""
        a = v.untyped_storage().data_ptr()
        return any(x is not None and any(y == a for y in _addresses(x)) for x in slots)

    def _aliased_later(self, slots, dst, i) -> bool:
        """True when a value computed before instruction ``i`` lives in the memory of ``dst`` (a view an
        earlier instruction made of a leaf) and is read after ``i``."""
        a = dst.untyped_storage().data_ptr()
        for s in range(self.nleaves, self.nslots):
            v = slots[s]
            if v is not None and self.last_use.get(s, -1) > i and any(x == a for x in _addresses(v)):
                return True
        return False

    def _destinations(self, leaf_vals, into):
        """instruction index -> destination tensor, for the roots that can be computed straight into
        their destination: the producing instruction writes into given memory, and no instruction
        after it reads a leaf that lives in the destination's memory (the producer itself may:
        an elementwise kernel reads each element before it writes it)."""
        out = {}
        for k, dst in into.items():
            slot = self.roots[k]
            i = self.writer.get(slot)
            if i is None or getattr(self.instrs[i][0], "_mimir_out", None) is None or self.roots.count(slot) != 1:
                continue
            a = dst.untyped_storage().data_ptr()
            safe = True
            for ls, v in enumerate(leaf_vals):
                if torch.is_tensor(v) and v.device.type != "meta" and v.untyped_storage().data_ptr() == a:
                    if self.last_use.get(ls, -1) > i:
                        safe = False
                    elif self.last_use.get(ls, -1) == i and (v.data_ptr() != dst.data_ptr() or tuple(v.shape) != tuple(dst.shape)
                                                             or v.stride() != dst.stride()):
                        safe = False      # the producer reads a shifted view of the memory it writes
            if safe:
                out[i] = dst
        return out


def _sole_owner(v) -> bool:
    """True when nothing but the running schedule can reach the memory of ``v``: the tensor spans its
    whole storage, no other tensor shares that storage (a view, a detached twin the caller kept) and
    no other Python reference to ``v`` exists besides the schedule's own (the caller's list of leaf
    values, this frame and the probe).  Memory the tensor does not own alone is never taken."""
    import sys
    if v.device.type == "meta" or not v.is_contiguous() or not v.numel():
        return False
    st = v.untyped_storage()
    if st.nbytes() != v.numel() * v.element_size():
        return False
    try:
        shared = torch._C._storage_Use_Count(st._cdata) > 2      # the tensor and this probe
    except Exception:  # noqa: BLE001 - without the counter, assume it is shared
        return False
    return not shared and sys.getrefcount(v) <= 4      # the leaf-value list, the two frames, the probe


def _addresses(v):
    if torch.is_tensor(v):
        if v.device.type != "meta":
            try:
                yield v.untyped_storage().data_ptr()
            except (NotImplementedError, RuntimeError):   # a transform's wrapper tensor
                return
    elif isinstance(v, (tuple, list)):
        for x in v:
            yield from _addresses(x)


def _device_of(slots, spec):
    for a in spec:
        if isinstance(a, _Ref) and torch.is_tensor(slots[a.slot]):
            return slots[a.slot].device
    return torch.device("cpu")


def _spec_slots(spec):
    for a in spec:
        if isinstance(a, _Ref):
            yield a.slot
        elif isinstance(a, (list, tuple)):
            yield from _spec_slots(a)


def _fill(spec, slots):
    out = []
    for a in spec:
        if isinstance(a, _Ref):
            out.append(slots[a.slot])
        elif isinstance(a, (list, tuple)):
            out.append(type(a)(_fill(a, slots)))
        else:
            out.append(a)
    return out


def _fn_key(fn):
    """Identity of an executable for the structural key: its code and the constants it closes over.
    A closed-over torch tensor (a frequency table, a mask) is keyed by identity: the cached program
    keeps the first closure alive, so the identity cannot be reused while the entry lives.  Returns
    None when a cell holds something that cannot be keyed (a lazy tensor, a list)."""
    from .core import Tensor
    code = getattr(fn, "__code__", None)
    if code is None:
        return None
    if getattr(fn, "_mimir_volatile", False):
        # the closure holds a per-call constant (a dropout or sampling seed): keyed by code only,
        # and a cached program takes this instruction's executable from the graph being run
        # (the reference keeps Attrs.Seed and Attrs.Value out of the key the same way)
        return (code, "volatile")
    cells = []
    for c in (fn.__closure__ or ()):
        v = c.cell_contents
        if isinstance(v, torch.Tensor):
            cells.append(("tensor", id(v)))
        elif isinstance(v, (list, tuple)) and all(isinstance(x, (int, float, bool, str, type(None))) for x in v):
            cells.append(tuple(v))          # a list of plain constants (split sizes, axes)
        elif isinstance(v, dict) and all(isinstance(k, str) and isinstance(x, (int, float, bool, str, type(None)))
                                         for k, x in v.items()):
            cells.append(tuple(sorted(v.items())))          # keyword constants of an elementwise op ({} most of the time)
        elif isinstance(v, (Tensor, list, dict, set)):
            return None
        elif callable(v) and hasattr(v, "__code__"):
            k = _fn_key(v)
            if k is None:
                return None
            cells.append(k)
        else:
            try:
                hash(v)
            except TypeError:
                return None
            cells.append(v)
    return (code, tuple(cells), getattr(fn, "__defaults__", None))


def _plain_key(a):
    if isinstance(a, (list, tuple)):
        return tuple(_plain_key(x) for x in a)
    if isinstance(a, torch.Tensor):
        return ("tensor", id(a))
    hash(a)
    return a


class _Walk:
    """One pass over the unrealized graph below the roots: topological order, reader counts."""

    def __init__(self, roots, memo, reuse_cached):
        from .core import Tensor, _flatten
        self.order, self.leaves = [], []          # interior nodes (post-order), leaf nodes
        self.readers = collections.Counter()
        self.index = {}                           # id(node) -> ("n", i) | ("l", i)
        for root in roots:
            if root._err is not None:
                raise root._err
            self.readers[id(root)] += 1
            stack = [(root, False)]
            while stack:
                t, expanded = stack.pop()
                if id(t) in self.index:
                    continue
                is_leaf = id(t) in memo or t._fn is None or (reuse_cached and t._val is not None)
                if is_leaf:
                    if id(t) not in memo and t._val is None:
                        if t._donated == 2:
                            raise E.ErrDonated("tensor was donated to an earlier schedule")
                        raise E.ErrNilTensor("tensor has neither a value nor a producer")
                    self.index[id(t)] = ("l", len(self.leaves))
                    self.leaves.append(t)
                    continue
                kids = [a for a in _flatten(t._args) if isinstance(a, Tensor)]
                if expanded:
                    self.index[id(t)] = ("n", len(self.order))
                    self.order.append(t)
                    continue
                stack.append((t, True))
                for a in kids:
                    self.readers[id(a)] += 1
                for a in reversed(kids):
                    if id(a) not in self.index:
                        stack.append((a, False))
        # a node pushed twice before its first expansion is counted once per reader, which is
        # what the planner wants; ``index`` makes every node appear once in ``order``


def _single_reader(w: _Walk, t) -> bool:
    return w.readers[id(t)] == 1 and w.index.get(id(t), ("l",))[0] == "n"


def _plan_fusion(w: _Walk):
    """Returns {id(consumer): (fn, args, kw, absorbed node)} for the patterns listed in the module
    docstring.  An absorbed node is not scheduled on its own."""
    from . import core as C
    out, absorbed = {}, set()
    for t in w.order:
        op = t._opname
        if op == "gelu" and (t._attrs or {}).get("approximate") == "tanh":
            (x,) = t._args
            a = x._attrs or {}
            if isinstance(x, C.Tensor) and x._opname == "linear" and a.get("act") == 0 and not a.get("residual") \
                    and _single_reader(w, x) and id(x) not in absorbed:
                out[id(t)] = (C._linear_run(1, a["bias"], False), x._args, {}, x)
                absorbed.add(id(x))
        elif op == "add":
            p, q = t._args
            for lin, res in ((p, q), (q, p)):
                a = (lin._attrs or {}) if isinstance(lin, C.Tensor) else {}
                if isinstance(lin, C.Tensor) and isinstance(res, C.Tensor) and lin._opname == "linear" \
                        and a.get("act") == 0 and not a.get("residual") and _single_reader(w, lin) \
                        and id(lin) not in absorbed and tuple(res.shape) == tuple(lin.shape) == tuple(t.shape) \
                        and res.dtype == lin.dtype == t.dtype and id(res) not in absorbed:
                    out[id(t)] = (C._linear_run(0, a["bias"], True), tuple(lin._args) + (res,), {}, lin)
                    absorbed.add(id(lin))
                    break
        elif op == "mul" and not (getattr(t.device, "kind", "") == "cpu" and t.dtype == torch.float32):
            # (float32 on the CPU: the elementwise fusion below takes the whole chain)
            p, q = t._args
            for act, up in ((p, q), (q, p)):
                if isinstance(act, C.Tensor) and isinstance(up, C.Tensor) and act._opname == "silu" \
                        and _single_reader(w, act) and id(act) not in absorbed \
                        and tuple(act.shape) == tuple(up.shape) == tuple(t.shape) and act.dtype == up.dtype:
                    out[id(t)] = (C._swiglu_run, (act._args[0], up), {}, act)
                    absorbed.add(id(act))
                    break
    _fuse_elementwise(w, out, absorbed)
    return out, absorbed


_MAX_CHAIN = 48       # instructions of one fused elementwise program
_MAX_INPUTS = 16


def _elementwise_name(t):
    """Name of the fusable elementwise op of node ``t`` (float32 on the CPU, plain arguments), or None."""
    from ..ops import fused_cpu as FC
    a = t._attrs or {}
    op = t._opname
    if op not in FC.OPS or t.dtype != torch.float32 or getattr(t.device, "kind", "") != "cpu" or t._sharding is not None:
        return None
    if a.get("kind") not in ("unary", "binary"):
        return None
    if a.get("kind") == "unary" and not a.get("plain", op == "gelu"):
        return None
    if op == "gelu" and a.get("approximate") != "tanh":
        return None
    return op


_FUSE_ELEMENTWISE = os.environ.get("MIMIR_FUSE", "1") not in ("0", "off", "false")


def set_elementwise_fusion(on: bool) -> bool:
    """Turns the fusion of elementwise chains on or off (``MIMIR_FUSE=0`` at start-up); returns the
    previous setting.  Cached programs are dropped, since they were planned under the other setting."""
    global _FUSE_ELEMENTWISE
    old, _FUSE_ELEMENTWISE = _FUSE_ELEMENTWISE, bool(on)
    clear_cache()
    return old


def _fuse_elementwise(w: _Walk, out, absorbed) -> None:
    """Chains (trees) of elementwise float32 CPU ops whose intermediate values have one reader become
    one fused program each: the root keeps its place in the schedule, the others are absorbed."""
    if not _FUSE_ELEMENTWISE:
        return
    from . import core as C
    from ..ops import fused_cpu as FC
    clusters = {}                      # id(root) -> members in topological order
    for t in w.order:
        if id(t) in absorbed or id(t) in out:
            continue
        name = _elementwise_name(t)
        if name is None:
            continue
        operands = [a for a in t._args if isinstance(a, C.Tensor)]
        if len(operands) != len(t._args) or not operands:
            continue
        n = t.numel()
        if any(a.dtype != torch.float32 or (tuple(a.shape) != tuple(t.shape) and a.numel() != 1) for a in operands):
            continue
        if n == 1 and any(tuple(a.shape) != tuple(t.shape) for a in operands):
            continue
        members = []
        for a in operands:
            sub = clusters.get(id(a))
            if sub is not None and _single_reader(w, a) and tuple(a.shape) == tuple(t.shape) \
                    and len(members) + len(sub) < _MAX_CHAIN:
                members += [m for m in sub if all(m is not x for x in members)]
                del clusters[id(a)]
        clusters[id(t)] = members + [t]
    by_id = {id(t): t for t in w.order}
    for root_id, members in clusters.items():
        if len(members) < 2:
            continue
        root = by_id[root_id]
        inside = {id(m): k for k, m in enumerate(members)}
        inputs, index = [], {}
        for m in members:
            for a in m._args:
                if id(a) not in inside and id(a) not in index:
                    index[id(a)] = len(inputs)
                    inputs.append(a)
        if len(inputs) > _MAX_INPUTS:
            continue
        n_in = len(inputs)
        reg = lambda a: n_in + inside[id(a)] if id(a) in inside else index[id(a)]   # noqa: E731
        instrs = []
        for m in members:
            ops = [reg(a) for a in m._args]
            instrs.append((m._opname, ops[0], ops[1] if len(ops) > 1 else None))
        prog = FC.Fused(instrs, n_in, root.shape)
        fn = _fused_executable(prog)
        out[root_id] = (fn, tuple(inputs), {}, None)
        for m in members[:-1]:
            absorbed.add(id(m))


def _fused_executable(prog):
    def run(*vals):
        return prog(*vals)

    def run_out(*vals, out):
        prog.into(*vals, out=out)
    run._mimir_out = run_out
    return run


def _compile(w: _Walk, roots, fusion, absorbed):
    from .core import Tensor
    nleaves = len(w.leaves)
    slot_of = {id(t): i for i, t in enumerate(w.leaves)}
    instrs, metas, nxt = [], [], nleaves

    def spec_of(args):
        sp = []
        for a in args:
            if isinstance(a, Tensor):
                sp.append(_Ref(slot_of[id(a)]))
            elif isinstance(a, (list, tuple)):
                sp.append(type(a)(spec_of(a)))
            else:
                sp.append(a)
        return tuple(sp)

    for i, t in enumerate(w.order):
        if id(t) in absorbed:
            continue
        if id(t) in fusion:
            fn, args, kw, _ = fusion[id(t)]
        else:
            fn, args, kw = t._fn, t._args, t._kw
        slot_of[id(t)] = nxt
        instrs.append((fn, spec_of(args), kw, nxt, i))
        metas.append((tuple(t.shape), t.dtype))
        nxt += 1
    return Program(instrs, nleaves, nxt, [slot_of[id(r)] for r in roots], len(fusion), metas)


def _structural_key(w: _Walk, roots):
    """Key of the walked graph, or None when some executable cannot be keyed."""
    from .core import Tensor
    parts = []
    try:
        for t in w.leaves:
            parts.append(("L", tuple(t.shape), t.dtype, repr(t.device), t._donated is True))   # a step that donates its batch has a program of its own
        for t in w.order:
            fk = _fn_key(t._fn)
            if fk is None:
                return None

            def arg_key(a):
                if isinstance(a, Tensor):
                    return w.index[id(a)]
                if isinstance(a, (list, tuple)):
                    return tuple(arg_key(x) for x in a)
                return _plain_key(a)
            parts.append((fk, tuple(arg_key(a) for a in t._args), tuple(sorted((k, _plain_key(v)) for k, v in t._kw.items())),
                          tuple(t.shape), t.dtype, w.readers[id(t)]))
        parts.append(tuple(w.index[id(r)] for r in roots))
        key = tuple(parts)
        hash(key)
        return key
    except TypeError:
        return None


def schedule(roots, memo=None, reuse_cached=True):
    """Plans (or finds) the program of ``roots`` and returns ``(program, walk)``; the caller runs it
    with the leaf values of *its* graph (``walk.leaves`` in order)."""
    memo = {} if memo is None else memo
    w = _Walk(roots, memo, reuse_cached)
    key = _structural_key(w, roots)
    if key is not None:
        prog = _CACHE.get(key)
        if prog is not None:
            _CACHE.move_to_end(key)
            _STATS["hits"] += 1
            return prog, w
    else:
        _STATS["uncacheable"] += 1
    fusion, absorbed = _plan_fusion(w)
    prog = _compile(w, roots, fusion, absorbed)
    _STATS["compiled"] += 1
    _STATS["fused"] += len(fusion)
    if key is not None:
        _CACHE[key] = prog
        while len(_CACHE) > _MAX_PROGRAMS:
            _CACHE.popitem(last=False)
    return prog, w
