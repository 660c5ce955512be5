"""Device groups and collectives (reference: tensor/group.go:57-478).

A ``Group`` is a set of ranks of one job (one process per device).  Collectives act
on axis 0 for all-gather / reduce-scatter like the reference; reductions are Sum,
Mean, Max, Min.  ``reduce_grads`` / ``all_reduce_grads`` / ``broadcast_params`` work on
lists of ``Param`` in buckets of about 25 MiB, last parameter first
(group.go:301-408), and are the NCCL baseline of the fused data-parallel kernel.
``cpus(n)`` runs a function on ``n`` CPU ranks (gloo) in child processes: the way
every distributed behaviour is tested without GPUs (tensor/group.go:57-72).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import core as C

_OPS = {"sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}
BUCKET_BYTES = 25 << 20


class Group:
    def __init__(self, ranks=None):
        if not dist.is_initialized():
            raise C.E.ErrDevice("torch.distributed is not initialised")
        self.ranks = list(ranks) if ranks is not None else list(range(dist.get_world_size()))
        self.pg = dist.new_group(self.ranks) if ranks is not None else None
        self.rank = dist.get_rank()
        self.size = len(self.ranks)
        self.traffic = {"all_reduce": 0, "broadcast": 0, "all_gather": 0, "reduce_scatter": 0, "reduce": 0, "bytes": 0}

    def _count(self, kind, t):
        self.traffic[kind] += 1
        self.traffic["bytes"] += t.numel() * t.element_size()

    def all_reduce(self, t: C.Tensor, op: str = "sum") -> C.Tensor:
        v = t.data().clone()
        self._count("all_reduce", v)
        dist.all_reduce(v, op=_OPS["sum" if op == "mean" else op], group=self.pg)
        return C.from_torch(v / self.size if op == "mean" else v)

    def broadcast(self, t: C.Tensor, root: int = 0) -> C.Tensor:
        v = t.data().clone()
        self._count("broadcast", v)
        dist.broadcast(v, self.ranks[root], group=self.pg)
        return C.from_torch(v)

    def all_gather(self, t: C.Tensor) -> C.Tensor:
        v = t.data().contiguous()
        self._count("all_gather", v)
        parts = [torch.empty_like(v) for _ in range(self.size)]
        dist.all_gather(parts, v, group=self.pg)
        return C.from_torch(torch.cat(parts, 0))

    def reduce_scatter(self, t: C.Tensor, op: str = "sum") -> C.Tensor:
        v = t.data().clone()
        self._count("reduce_scatter", v)
        if v.shape[0] % self.size:
            raise C.E.ErrShape("reduce_scatter: axis 0 does not divide by the group size")
        dist.all_reduce(v, op=_OPS["sum" if op == "mean" else op], group=self.pg)
        out = v.chunk(self.size, 0)[self.ranks.index(self.rank)].contiguous()
        return C.from_torch(out / self.size if op == "mean" else out)

    # -- gradient / parameter buckets
    def _buckets(self, tensors):
        bucket, size = [], 0
        for t in reversed(tensors):
            bucket.append(t)
            size += t.numel() * t.element_size()
            if size >= BUCKET_BYTES:
                yield bucket
                bucket, size = [], 0
        if bucket:
            yield bucket

    def all_reduce_grads(self, params, op: str = "mean") -> None:
        grads = [p._grad for p in params if p._grad is not None]
        for bucket in self._buckets(grads):
            flat = torch.cat([g.reshape(-1) for g in bucket])
            self._count("all_reduce", flat)
            dist.all_reduce(flat, op=_OPS["sum" if op == "mean" else op], group=self.pg)
            if op == "mean":
                flat /= self.size
            off = 0
            for g in bucket:
                g.copy_(flat[off: off + g.numel()].view_as(g))
                off += g.numel()

    def reduce_grads(self, params, root: int = 0, op: str = "mean") -> None:
        grads = [p._grad for p in params if p._grad is not None]
        for bucket in self._buckets(grads):
            flat = torch.cat([g.reshape(-1) for g in bucket])
            self._count("reduce", flat)
            dist.reduce(flat, self.ranks[root], op=_OPS["sum" if op == "mean" else op], group=self.pg)
            if op == "mean":
                flat /= self.size
            if self.rank == self.ranks[root]:
                off = 0
                for g in bucket:
                    g.copy_(flat[off: off + g.numel()].view_as(g))
                    off += g.numel()

    def broadcast_params(self, params, root: int = 0) -> None:
        for bucket in self._buckets([p._data for p in params]):
            flat = torch.cat([t.reshape(-1) for t in bucket])
            self._count("broadcast", flat)
            dist.broadcast(flat, self.ranks[root], group=self.pg)
            off = 0
            for t in bucket:
                t.copy_(flat[off: off + t.numel()].view_as(t))
                off += t.numel()
        for p in params:
            p._version += 1

    def close(self):
        if self.pg is not None:
            dist.destroy_process_group(self.pg)


def _cpu_rank(rank, world, port, fn, args, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    C.set_default_device(C.CPU())
    try:
        queue.put((rank, fn(Group(), *args)))
    except BaseException as e:  # the parent re-raises it instead of waiting for a result
        queue.put((rank, _Failed(f"{type(e).__name__}: {e}")))
        raise
    finally:
        dist.destroy_process_group()


class _Failed:
    def __init__(self, why):
        self.why = why


def cpus(n: int, fn, *args, port: int = 29671):
    """Runs ``fn(group, *args)`` on ``n`` CPU ranks; returns the results ordered by rank."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_cpu_rank, args=(r, n, port, fn, args, q)) for r in range(n)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(n):
            r, v = q.get(timeout=120)
            if isinstance(v, _Failed):
                raise C.E.ErrDevice(f"rank {r} failed: {v.why}")
            out[r] = v
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.terminate()
    return [out[r] for r in range(n)]
